"""Computed-torque control (control mode 3) in the CPU oracle against closed forms (the reference's
ApplyDynamicsDriveKernel, ops/articulation.cu:1315-1418).  On a fixed-base arm without contacts, joint damping or
force limits the controller's command makes the joint accelerations equal its right-hand side a* + kp (q* - q) +
kd (qd* - qd) whatever the pose and velocity: the mass matrix and the velocity-product forces cancel."""
import numpy as np

from nuka import templates as T


def arm_world(oracle, E, seed=0):
    w = oracle.World(T.arm7(0).blob(), E)
    st = T.arm7_state(E, seed)
    w.set("q", st["q"]); w.set("qdot", st["qdot"])
    w.refresh()
    w.set_control_mode(3)
    return w, st


def test_accelerations_equal_the_controller_right_hand_side(oracle):
    E, L = 16, 8
    w, st = arm_world(oracle, E)
    rng = np.random.Generator(np.random.PCG64(7))
    acc = np.zeros((E, L), np.float32); acc[:, 1:] = rng.normal(0, 2.0, size=(E, L - 1))
    target = st["q"] + rng.normal(0, 0.2, size=(E, L)).astype(np.float32)
    vtarget = np.zeros((E, L), np.float32); vtarget[:, 1:] = rng.normal(0, 0.5, size=(E, L - 1))
    kp = np.full((E, L), 25.0, np.float32); kd = np.full((E, L), 3.0, np.float32)
    w.set("acceleration_target", acc); w.set("drive_target", target); w.set("velocity_target", vtarget)
    w.set("drive_stiffness", kp); w.set("drive_damping", kd)
    q0, qd0 = w.get("q", L).copy(), w.get("qdot", L).copy()
    want = acc + kp * (target - q0) + kd * (vtarget - qd0)
    w.step(1)
    assert not w.get("env_status", 1).any()
    dt = 1.0 / 500.0
    got = (w.get("qdot", L) - qd0) / dt
    scale = np.abs(want[:, 1:]).max()
    assert np.abs(got[:, 1:] - want[:, 1:]).max() / scale < 2e-3          # fp32 through M^-1 and its inverse, over dt


def test_zero_gains_hold_the_arm_against_gravity(oracle):
    """a* = 0 with zero gains is pure bias compensation: a moving arm keeps its joint rates over a step."""
    E, L = 8, 8
    w, st = arm_world(oracle, E, seed=3)
    zero = np.zeros((E, L), np.float32)
    w.set("drive_stiffness", zero); w.set("drive_damping", zero)
    qd0 = w.get("qdot", L).copy()
    w.step(1)
    assert np.abs(w.get("qdot", L) - qd0).max() < 2e-4


def test_force_limit_clamps_the_command(oracle):
    E, L = 4, 8
    w, st = arm_world(oracle, E)
    acc = np.zeros((E, L), np.float32); acc[:, 1:] = 500.0                    # asks for far more than the limit allows
    w.set("acceleration_target", acc)
    w.set("drive_force_limit", np.full((E, L), 0.5, np.float32))
    w.set("drive_stiffness", np.zeros((E, L), np.float32)); w.set("drive_damping", np.zeros((E, L), np.float32))
    w.step(1)
    applied = w.get("actuator_applied", L)
    assert np.abs(applied[:, 1:]).max() <= 0.5 * (1 + 1e-5) and np.abs(applied[:, 1:]).max() > 0.49


def test_rejected_input_raises_the_control_status(oracle):
    E, L = 4, 8
    w, st = arm_world(oracle, E)
    acc = np.zeros((E, L), np.float32); acc[2, 3] = np.nan
    w.set("acceleration_target", acc)
    w.step(1)
    status = w.get("env_status", 1)[:, 0]
    assert status[2] & (1 << 10) and not (status[[0, 1, 3]] & (1 << 10)).any()
