"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on the same seeded inputs and
against the committed golden fixtures.

Tolerances (fp32): mass matrices, accelerations and single-step post-solve velocities within 1e-5 of the
field's largest magnitude; 100-step contact-free trajectories within 1e-4; candidate pair lists bit-exact.
"""
import os

import numpy as np
import pytest

import nuka
from nuka import Field as F, templates as T

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-12))


def quad_inputs(E, seed=0):
    st = T.quadruped_state(E, seed)
    rng = np.random.Generator(np.random.PCG64(7 + seed))
    qdot = np.zeros((E, 13), np.float32)
    qdot[:, 1:] = rng.normal(0, 0.5, size=(E, 12))
    lv = np.zeros((E, 13, 6), np.float32)
    lv[:, 0, :] = rng.normal(0, 0.3, size=(E, 6))
    return st["q"], qdot, st["base_pose"], lv.reshape(E, -1)


def make_pair(device, oracle, tb, E, state):
    blob = tb.blob()
    w = nuka.World.create_from_template(device, blob, E)
    o = oracle.World(blob, E)
    names = {"q": F.JOINT_POSITION, "qdot": F.JOINT_VELOCITY, "base_pose": F.BASE_POSE, "link_velocity": F.LINK_VELOCITY,
             "body_pose": F.RIGID_BODY_TRANSFORM, "body_linear_velocity": F.BODY_LINEAR_VELOCITY}
    for k, v in state.items():
        w.upload(names[k], v)
        o.set(k, v.reshape(E, -1))
    w.forward_kinematics()
    o.refresh()
    return w, o


def test_arm7_dynamics_and_trajectory(device, oracle):
    E = 64
    st = T.arm7_state(E, 0)
    w, o = make_pair(device, oracle, T.arm7(0), E, st)
    assert rel(w.download(F.ARTICULATION_LINK_POSE), o.get("link_pose", 56)) < 1e-6
    w.run_stage(1); o.dynamics(False)
    assert rel(w.download(F.MASS_MATRIX), o.get("mass_matrix", 49)) < 1e-5
    assert rel(w.download(F.JOINT_ACCELERATION), o.get("qddot", 8)) < 2e-5
    w.step_n(100); o.step(100)
    assert rel(w.download(F.JOINT_POSITION), o.get("q", 8)) < 1e-4
    assert rel(w.download(F.JOINT_VELOCITY), o.get("qdot", 8)) < 1e-4
    assert w.download(F.ENV_STATUS).max() == 0
    w.destroy()


def test_arm7_golden(device):
    g = np.load(os.path.join(GOLDEN, "arm7_seed0.npz"))
    w = nuka.World.create_from_template(device, T.arm7(0).blob(), 4)
    w.upload(F.JOINT_POSITION, g["q_in"]); w.upload(F.JOINT_VELOCITY, g["qdot_in"]); w.forward_kinematics()
    w.run_stage(1)
    assert rel(w.download(F.MASS_MATRIX), g["mass"]) < 1e-5 and rel(w.download(F.JOINT_ACCELERATION), g["qdd"]) < 2e-5
    w.step_n(100)
    assert rel(w.download(F.JOINT_POSITION), g["q_100"]) < 1e-4
    w.destroy()


def test_quadruped_stages(device, oracle):
    E = 256
    q, qdot, base, lv = quad_inputs(E)
    state = {"q": q, "qdot": qdot, "base_pose": base, "link_velocity": lv}
    w, o = make_pair(device, oracle, T.quadruped(0), E, state)
    assert rel(w.download(F.RIGID_BODY_TRANSFORM), o.get("body_pose", 98)) < 1e-6
    w.run_stage(1); o.dynamics(False)
    assert rel(w.download(F.MASS_MATRIX), o.get("mass_matrix", 324)) < 1e-5
    assert rel(w.download(F.JOINT_ACCELERATION), o.get("qddot", 13)) < 2e-5
    w.run_stage(2); o.collide()
    assert np.array_equal(w.download(F.PAIR_COUNT), o.get("pair_count", 1))
    assert np.array_equal(w.download(F.CANDIDATE_PAIRS), o.get("candidate_pairs", 16))      # bit-exact, canonical order
    assert np.array_equal(w.download(F.CONTACT_COUNT), o.get("contact_count", 8))
    assert rel(w.download(F.CONTACT_POINT), o.get("contact_point", 96)) < 1e-5
    assert rel(w.download(F.CONTACT_DEPTH), o.get("contact_depth", 32)) < 1e-4
    w.destroy()


def test_quadruped_single_step_post_solve(device, oracle):
    E = 256
    q, qdot, base, lv = quad_inputs(E)
    state = {"q": q, "qdot": qdot, "base_pose": base, "link_velocity": lv}
    w, o = make_pair(device, oracle, T.quadruped(0), E, state)
    w.step(); o.step(1)
    assert o.get("contact_points", 1).sum() > E          # the case really has contacts
    assert rel(w.download(F.JOINT_VELOCITY), o.get("qdot", 13)) < 1e-5
    assert rel(w.download(F.LINK_VELOCITY), o.get("link_velocity", 78)) < 1e-5
    assert rel(w.download(F.BASE_POSE), o.get("base_pose", 7)) < 1e-6
    assert rel(w.download(F.JOINT_POSITION), o.get("q", 13)) < 1e-6
    assert np.array_equal(w.download(F.SOLVER_SWEEPS)[:, 0], o.get("solver_sweeps", 1)[:, 0])
    assert w.download(F.ENV_STATUS).max() == 0
    w.destroy()


def test_quadruped_golden(device):
    g = np.load(os.path.join(GOLDEN, "quadruped_seed0.npz"))
    w = nuka.World.create_from_template(device, T.quadruped(0).blob(), 4)
    for f, k in ((F.JOINT_POSITION, "q_in"), (F.JOINT_VELOCITY, "qdot_in"), (F.BASE_POSE, "base_in"), (F.LINK_VELOCITY, "link_vel_in")):
        w.upload(f, g[k])
    w.forward_kinematics()
    w.run_stage(2)
    assert np.array_equal(w.download(F.CANDIDATE_PAIRS), g["pairs"]) and np.array_equal(w.download(F.CONTACT_COUNT), g["contact_count"])
    w.step()
    assert rel(w.download(F.JOINT_VELOCITY), g["qdot_1"]) < 1e-5 and rel(w.download(F.LINK_VELOCITY), g["link_vel_1"]) < 1e-5
    w.destroy()


def test_quadruped_no_contact_trajectory(device, oracle):
    """100 steps without contacts (no ground plane): 1e-4."""
    E = 64
    tb = T.quadruped(0)
    tb.bodies = [b for b in tb.bodies if b["kind"] != T.PLANE]
    q, qdot, base, lv = quad_inputs(E, 1)
    w, o = make_pair(device, oracle, tb, E, {"q": q, "qdot": qdot * 0.2, "base_pose": base, "link_velocity": lv})
    w.step_n(100); o.step(100)
    assert rel(w.download(F.JOINT_POSITION), o.get("q", 13)) < 1e-4
    assert rel(w.download(F.BASE_POSE), o.get("base_pose", 7)) < 1e-4
    w.destroy()


def test_quadruped_stands_for_a_second(device):
    """Size-independent property at the benchmark size: all 4096 robots keep standing on their feet."""
    E = 4096
    w = nuka.World.create_from_template(device, T.quadruped(0).blob(), E)
    st = T.quadruped_state(E, 0)
    w.upload(F.JOINT_POSITION, st["q"]); w.upload(F.BASE_POSE, st["base_pose"]); w.forward_kinematics()
    w.step_n(200)
    base = w.download(F.BASE_POSE)
    assert np.isfinite(base).all() and base[:, 2].min() > 0.2 and base[:, 2].max() < 0.4
    assert np.allclose(np.linalg.norm(base[:, 3:], axis=1), 1.0, atol=1e-4)
    assert w.download(F.ENV_STATUS).max() == 0
    w.destroy()


def test_quadruped_contact_trajectory_tracks_the_oracle(device, oracle):
    """Standing quadrupeds in contact: warm-started multi-step trajectories stay on the oracle's (20 steps,
    positions within 1e-4 of the largest magnitude), with the same sweep counts."""
    E = 256
    st = T.quadruped_state(E, 3)
    w, o = make_pair(device, oracle, T.quadruped(0), E, {"q": st["q"], "base_pose": st["base_pose"]})
    w.step_n(20); o.step(20)
    assert rel(w.download(F.JOINT_POSITION), o.get("q", 13)) < 1e-4
    assert rel(w.download(F.BASE_POSE), o.get("base_pose", 7)) < 1e-4
    assert np.mean(w.download(F.SOLVER_SWEEPS) == o.get("solver_sweeps", 1)) > 0.98
    assert w.download(F.ENV_STATUS).max() == 0
    w.destroy()


def test_benchmark_size_runs_are_reproducible(device):
    """Two runs of the 4096-env workload from the same inputs end in byte-identical state (no data races)."""
    E = 4096
    blob = T.quadruped(0).blob()
    st = T.quadruped_state(E, 0)
    ends = []
    for _ in range(2):
        w = nuka.World.create_from_template(device, blob, E)
        w.upload(F.JOINT_POSITION, st["q"]); w.upload(F.BASE_POSE, st["base_pose"]); w.forward_kinematics()
        w.step_n(50)
        ends.append((w.download(F.JOINT_POSITION).tobytes(), w.download(F.BASE_POSE).tobytes(), w.download(F.JOINT_VELOCITY).tobytes()))
        w.destroy()
    assert ends[0] == ends[1]


def test_env_shards_equal_the_whole_batch(device):
    """The property multi-GPU runs rest on, at configs[4]'s per-GPU size: 8192 quadruped + 4 boxes envs stepped as one
    world and as two 4096-env shards (contiguous env ranges, as nuka.shard.env_range hands them out) end in
    byte-identical state, so a sharded run equals the single-world run env for env."""
    from nuka import shard
    E, parts = 8192, 2
    blob = T.quadruped(0, boxes=4).blob()
    st = T.quadruped_state(E, 4)
    fields = (F.JOINT_POSITION, F.JOINT_VELOCITY, F.BASE_POSE, F.RIGID_BODY_TRANSFORM, F.BODY_LINEAR_VELOCITY, F.CONTACT_COUNT)

    def run(lo, hi):
        w = nuka.World.create_from_template(device, blob, hi - lo)
        w.upload(F.JOINT_POSITION, st["q"][lo:hi]); w.upload(F.BASE_POSE, st["base_pose"][lo:hi]); w.forward_kinematics()
        w.step_n(30)
        out = [w.download(f).copy() for f in fields]
        w.destroy()
        return out

    whole = run(0, E)
    for rank in range(parts):
        lo, hi = shard.env_range(rank, parts, E)
        part = run(lo, hi)
        for f, a, b in zip(fields, whole, part):
            assert np.array_equal(a[lo:hi], b), (rank, f)


def test_free_boxes_land_like_the_oracle(device, oracle):
    """Six free boxes falling onto a plane (the free rigid-body path: gyroscopic integration, box-plane and
    box-box manifolds, 6-coordinate solver blocks): candidate pairs and contact counts bit-exact, poses within
    1e-4 through the first landings."""
    E = 64
    st = T.box_pile_state(E, 2, count=6)
    w, o = make_pair(device, oracle, T.box_pile(2, count=6), E, {"body_pose": st["body_pose"]})
    B, S = 7, w.info.contact_slots_per_env
    for k in (1, 14, 25):
        w.step_n(k); o.step(k)
        pc = w.download(F.PAIR_COUNT)
        assert np.array_equal(pc, o.get("pair_count", 1))
        live = np.arange(S)[None, :] < pc                      # slots past the pair count are unspecified
        gp = w.download(F.CANDIDATE_PAIRS).reshape(E, S, 2)
        op = o.get("candidate_pairs", 2 * S).reshape(E, S, 2)
        assert np.array_equal(gp[live], op[live])
        assert np.array_equal(w.download(F.CONTACT_COUNT)[live], o.get("contact_count", S)[live])
        assert rel(w.download(F.RIGID_BODY_TRANSFORM), o.get("body_pose", 7 * B)) < 1e-4
    assert w.download(F.PAIR_COUNT).max() > 0 and w.download(F.ENV_STATUS).max() == 0
    w.destroy()


def test_full_box_pile_of_configs_3(device, oracle):
    """configs[3]'s env at full size: 48 free boxes over a plane, 288 candidate slots, a contact-point capacity of
    288 carried by the template.  Pair lists and contact counts bit-exact and poses within 1e-4 through the first
    landings (after which a tumbling pile amplifies rounding differences)."""
    E, count = 16, 48
    st = T.box_pile_state(E, 0, count=count)
    w, o = make_pair(device, oracle, T.box_pile(0, count=count), E, {"body_pose": st["body_pose"]})
    B, S = count + 1, w.info.contact_slots_per_env
    assert S == 6 * count
    for k in (1, 19):
        w.step_n(k); o.step(k)
        pc = w.download(F.PAIR_COUNT)
        assert np.array_equal(pc, o.get("pair_count", 1))
        live = np.arange(S)[None, :] < pc
        assert np.array_equal(w.download(F.CANDIDATE_PAIRS).reshape(E, S, 2)[live], o.get("candidate_pairs", 2 * S).reshape(E, S, 2)[live])
        assert np.array_equal(w.download(F.CONTACT_COUNT)[live], o.get("contact_count", S)[live])
        assert rel(w.download(F.RIGID_BODY_TRANSFORM), o.get("body_pose", 7 * B)) < 1e-4
    assert w.download(F.CONTACT_COUNT).sum() > 0 and w.download(F.ENV_STATUS).max() == 0
    w.destroy()


def test_quadruped_with_free_boxes(device, oracle):
    """configs[4]'s env: the quadruped plus four free boxes (articulated and rigid blocks in one solve)."""
    E = 64
    st = T.quadruped_state(E, 4)
    w, o = make_pair(device, oracle, T.quadruped(0, boxes=4), E, {"q": st["q"], "base_pose": st["base_pose"]})
    w.step_n(30); o.step(30)
    assert rel(w.download(F.JOINT_POSITION), o.get("q", 13)) < 1e-4
    assert rel(w.download(F.BASE_POSE), o.get("base_pose", 7)) < 1e-4
    assert rel(w.download(F.RIGID_BODY_TRANSFORM), o.get("body_pose", 18 * 7)) < 1e-4
    assert np.array_equal(w.download(F.CONTACT_COUNT), o.get("contact_count", w.info.contact_slots_per_env))
    assert w.download(F.ENV_STATUS).max() == 0
    w.destroy()


def _mixed_shapes():
    """Two capsules, two spheres and a box over a plane; filter bits keep the (unsupported) capsule-box pair out."""
    from nuka.templates import BOX, CAPSULE, SPHERE, TemplateBuilder, box_inertia
    tb = TemplateBuilder(dt=1 / 240.0, vel_iters=8, max_contacts=16)
    cap_i = (0.004, 0.004, 0.001)
    tb.add_free_body((CAPSULE, 0.04, 0.12), 1.0, cap_i, (0.0, 0.0, 0.10, 0.7071068, 0, 0.7071068, 0), mu=0.6)
    tb.add_free_body((CAPSULE, 0.04, 0.12), 1.0, cap_i, (0.02, 0.0, 0.22, 0.5, 0.5, 0.5, 0.5), mu=0.6)
    tb.add_free_body((SPHERE, 0.05), 0.5, (0.0005,) * 3, (0.05, 0.03, 0.36, 1, 0, 0, 0), mu=0.6, conaffinity=9)
    tb.add_free_body((SPHERE, 0.05), 0.5, (0.0005,) * 3, (0.30, 0.0, 0.30, 1, 0, 0, 0), mu=0.6, conaffinity=9)
    tb.add_free_body((BOX, 0.06, 0.06, 0.06), 1.5, box_inertia(1.5, (0.12,) * 3), (0.31, 0.01, 0.10, 1, 0, 0, 0), mu=0.6,
                     contype=8, conaffinity=16)
    tb.add_plane(0.0, mu=0.8, conaffinity=9)
    return tb


def test_every_analytic_pair_kind_matches_the_oracle(device, oracle):
    """sphere-plane, sphere-box, capsule-plane, capsule-sphere, capsule-capsule and box-plane manifolds in one
    world: pair lists and contact counts bit-exact, poses within 1e-4; live contact points within 1e-4 while the
    poses still agree to 1e-6 (closest points of near-parallel capsules amplify pose differences later on)."""
    E, steps = 32, (1, 40, 40)
    tb = _mixed_shapes()
    rng = np.random.Generator(np.random.PCG64(3))
    pose = np.tile(tb.arrays()["body_pose0"].reshape(1, 6, 7), (E, 1, 1)).astype(np.float32)
    pose[:, :5, :3] += rng.uniform(-0.01, 0.01, size=(E, 5, 3)).astype(np.float32)
    w, o = make_pair(device, oracle, tb, E, {"body_pose": pose})
    S = w.info.contact_slots_per_env
    kinds = tb.arrays()["shape_kind"]
    seen = set()
    for k in steps:
        w.step_n(k); o.step(k)
        pc = w.download(F.PAIR_COUNT)
        assert np.array_equal(pc, o.get("pair_count", 1))
        live = np.arange(S)[None, :] < pc
        gp = w.download(F.CANDIDATE_PAIRS).reshape(E, S, 2)
        assert np.array_equal(gp[live], o.get("candidate_pairs", 2 * S).reshape(E, S, 2)[live])
        cc = w.download(F.CONTACT_COUNT)
        assert np.array_equal(cc[live], o.get("contact_count", S)[live])
        points = (np.arange(4)[None, None, :] < cc[:, :, None]) & live[:, :, None]
        pose_error = rel(w.download(F.RIGID_BODY_TRANSFORM), o.get("body_pose", 42))
        assert pose_error < 1e-4
        if points.any() and pose_error < 1e-6:
            gpt = w.download(F.CONTACT_POINT).reshape(E, S, 4, 3)[points]
            opt = o.get("contact_point", 12 * S).reshape(E, S, 4, 3)[points]
            assert np.abs(gpt - opt).max() < 1e-4
        for env, slot in zip(*np.nonzero((cc > 0) & live)):
            seen.add((int(kinds[gp[env, slot, 0]]), int(kinds[gp[env, slot, 1]])))
    assert {(0, 2), (1, 0), (1, 1), (1, 3), (2, 3)} <= seen        # the sphere-plane kind shows up later in time
    assert w.download(F.ENV_STATUS).max() == 0
    w.destroy()


def test_go2_scene_template(device, oracle):
    """The reference's Go2 scene, cooked by nuka.nks into tests/golden/go2.nkt (23 collision shapes on 13 links,
    joint limits, rotated inertial frames): per-stage and trajectory parity with the oracle, and it keeps standing."""
    with open(os.path.join(GOLDEN, "go2.nkt"), "rb") as f:
        blob = f.read()
    E = 32
    w = nuka.World.create_from_template(device, blob, E)
    o = oracle.World(blob, E)
    rng = np.random.Generator(np.random.PCG64(11))
    q = w.download(F.JOINT_POSITION)
    q[:, 1:] += rng.uniform(-0.05, 0.05, size=(E, 12)).astype(np.float32)
    w.upload(F.JOINT_POSITION, q); o.set("q", q)
    w.forward_kinematics(); o.refresh()
    B, S = w.info.bodies_per_env, w.info.contact_slots_per_env
    assert (B, w.info.dofs_per_env) == (24, 18)
    assert rel(w.download(F.RIGID_BODY_TRANSFORM), o.get("body_pose", 7 * B)) < 1e-6
    w.run_stage(1); o.dynamics(False)
    assert rel(w.download(F.MASS_MATRIX), o.get("mass_matrix", 18 * 18)) < 1e-5
    w.step_n(20); o.step(20)
    assert rel(w.download(F.JOINT_POSITION), o.get("q", 13)) < 1e-4
    assert rel(w.download(F.BASE_POSE), o.get("base_pose", 7)) < 1e-4
    pc = w.download(F.PAIR_COUNT)
    assert np.array_equal(pc, o.get("pair_count", 1))
    live = np.arange(S)[None, :] < pc
    assert np.array_equal(w.download(F.CONTACT_COUNT)[live], o.get("contact_count", S)[live])
    w.step_n(400)
    base = w.download(F.BASE_POSE)
    assert (base[:, 2] > 0.22).all() and (base[:, 2] < 0.33).all() and (np.abs(base[:, 4:6]) < 0.1).all()
    assert w.download(F.ENV_STATUS).max() == 0
    w.destroy()


@pytest.mark.parametrize("mode", [1, 2, 5])
def test_torque_and_velocity_control_modes(device, oracle, mode):
    """control_mode 1 (the target field is a joint torque), 2 (velocity servo with gain kp) and 5 (actuator: torque
    command inside a torque-speed envelope, written through TORQUE_INPUT): trajectories of the standing quadruped
    under each mode follow the oracle's."""
    E = 48
    tb = T.quadruped(0)
    blob = tb.blob()
    w = nuka.World.create_from_template(device, blob, E, control_mode=mode)
    o = oracle.World(blob, E)
    o.set_control_mode(mode)
    st = T.quadruped_state(E, 6)
    rng = np.random.Generator(np.random.PCG64(20 + mode))
    target = np.zeros((E, 13), np.float32)
    vt = np.zeros((E, 13), np.float32)
    extra = []
    if mode == 1:
        target[:, 1:] = rng.uniform(-3.0, 3.0, size=(E, 12))          # joint torques, N m
    elif mode == 5:
        target[:, 1:] = rng.uniform(-6.0, 6.0, size=(E, 12))          # commands beyond the 4 N m stall torque
        limit = np.full((E, 13), 4.0, np.float32)
        noload = np.zeros((E, 13), np.float32)
        noload[:, 1:] = rng.uniform(1.0, 3.0, size=(E, 12))           # rad/s
        noload[:, 1] = 0.0                                            # one joint without a speed envelope
        extra = [(F.DRIVE_FORCE_LIMIT, "drive_force_limit", limit), (F.ACTUATOR_NOLOAD_SPEED, "noload_speed", noload)]
    else:
        vt[:, 1:] = rng.uniform(-0.5, 0.5, size=(E, 12))              # joint velocity targets, rad/s
    for world_set, oracle_name, value in ((F.JOINT_POSITION, "q", st["q"]), (F.BASE_POSE, "base_pose", st["base_pose"]),
                                          (F.TORQUE_INPUT if mode == 5 else F.DRIVE_TARGET, "drive_target", target),
                                          (F.VELOCITY_TARGET, "velocity_target", vt), *extra):
        w.upload(world_set, value); o.set(oracle_name, value.reshape(E, -1))
    w.forward_kinematics(); o.refresh()
    w.step_n(1); o.step(1)
    # the velocity servo (gain 40 on every joint) makes the step stiffer than the PD hold: 5e-5 there, 2e-5 for torques
    assert rel(w.download(F.JOINT_VELOCITY), o.get("qdot", 13)) < (5e-5 if mode == 2 else 2e-5)
    w.step_n(19); o.step(19)
    assert rel(w.download(F.JOINT_POSITION), o.get("q", 13)) < 1e-4
    assert rel(w.download(F.BASE_POSE), o.get("base_pose", 7)) < 1e-4
    assert w.download(F.ENV_STATUS).max() == 0
    moved = np.abs(w.download(F.JOINT_POSITION)[:, 1:] - st["q"][:, 1:]).max()
    assert moved > 0.01                                               # the commands really drive the joints
    w.destroy()


def test_humanoid_35_coordinates(device, oracle):
    """configs[2]'s articulation: 30 links, 35 coordinates (two per warp lane), capsules on a plane and limb-limb
    self-contact: mass matrix, accelerations, a single step and a short trajectory against the oracle.  Envs whose
    solve stops at the sweep limit (crossed legs pressing into each other) carry an unconverged state forward, which
    amplifies rounding differences, so the 2e-4 trajectory bound applies to the envs that converged in every step
    and a 1e-2 bound to the rest."""
    E = 24
    tb = T.humanoid(0)
    st = T.humanoid_state(E, 1)
    rng = np.random.Generator(np.random.PCG64(5))
    qdot = np.zeros((E, 30), np.float32)
    qdot[:, 1:] = rng.normal(0, 0.3, size=(E, 29))
    w, o = make_pair(device, oracle, tb, E, {"q": st["q"], "qdot": qdot})
    assert w.info.dofs_per_env == 35
    assert rel(w.download(F.ARTICULATION_LINK_POSE), o.get("link_pose", 30 * 7)) < 1e-6
    w.run_stage(1); o.dynamics(False)
    assert rel(w.download(F.MASS_MATRIX), o.get("mass_matrix", 35 * 35)) < 1e-5
    assert rel(w.download(F.JOINT_ACCELERATION), o.get("qddot", 30)) < 5e-5
    w.step_n(1); o.step(1)
    assert rel(w.download(F.JOINT_VELOCITY), o.get("qdot", 30)) < 5e-5
    assert np.array_equal(w.download(F.PAIR_COUNT), o.get("pair_count", 1))
    S = w.info.contact_slots_per_env
    limit = w.get_velocity_iterations()
    converged = np.ones(E, bool)
    self_contacts = 0
    differing = 0
    for _ in range(19):
        w.step_n(1); o.step(1)
        sweeps = w.download(F.SOLVER_SWEEPS).reshape(E)
        # the sweep count is a data-dependent stopping decision at a 1e-5 residual threshold: last-bit differences between the
        # two fp32 evaluations may move it in a rare env, which then counts as not converged for the tight comparison below
        same = sweeps == o.get("solver_sweeps", 1).reshape(E)
        differing += int((~same).sum())
        converged &= (sweeps < limit) & same
        cc = w.download(F.CONTACT_COUNT)
        assert np.array_equal(cc, o.get("contact_count", S))
        self_contacts += int(((w.download(F.CANDIDATE_PAIRS).reshape(E, S, 2)[:, :, 1] != 30) & (cc > 0)).sum())
    assert self_contacts > 0 and converged.sum() >= E // 2 and differing <= E // 4
    gq, oq = w.download(F.JOINT_POSITION), o.get("q", 30).reshape(E, 30)
    gb, ob = w.download(F.BASE_POSE), o.get("base_pose", 7).reshape(E, 7)
    assert rel(gq[converged], oq[converged]) < 2e-4 and rel(gb[converged], ob[converged]) < 2e-4
    assert rel(gq, oq) < 1e-2 and rel(gb, ob) < 1e-2
    assert w.download(F.ENV_STATUS).max() == 0 and o.get("env_status", 1).max() == 0
    w.destroy()


def test_computed_torque_control(device, oracle):
    """control_mode 3 (the reference's ApplyDynamicsDriveKernel, ComputedTorque branch): the commanded joint accelerations
    a* + kp (q* - q) + kd (qd* - qd) are realised through H = (S M^-1 S^T)^-1 with bias compensation.  A fixed-base arm
    without contacts must reproduce the closed form (accelerations equal the right-hand side); a standing quadruped with
    foot contacts and force limits follows the oracle."""
    E, L = 32, 8
    blob = T.arm7(0).blob()
    w = nuka.World.create_from_template(device, blob, E, control_mode=3)
    o = oracle.World(blob, E)
    o.set_control_mode(3)
    st = T.arm7_state(E, 0)
    rng = np.random.Generator(np.random.PCG64(7))
    acc = np.zeros((E, L), np.float32); acc[:, 1:] = rng.normal(0, 2.0, size=(E, L - 1))
    target = (st["q"] + rng.normal(0, 0.2, size=(E, L))).astype(np.float32)
    vt = np.zeros((E, L), np.float32); vt[:, 1:] = rng.normal(0, 0.5, size=(E, L - 1))
    kp, kd = np.full((E, L), 25.0, np.float32), np.full((E, L), 3.0, np.float32)
    for field, name, value in ((F.JOINT_POSITION, "q", st["q"]), (F.JOINT_VELOCITY, "qdot", st["qdot"]), (F.ACCELERATION_TARGET, "acceleration_target", acc),
                               (F.DRIVE_TARGET, "drive_target", target), (F.VELOCITY_TARGET, "velocity_target", vt),
                               (F.DRIVE_STIFFNESS, "drive_stiffness", kp), (F.DRIVE_DAMPING, "drive_damping", kd)):
        w.upload(field, value); o.set(name, value)
    w.forward_kinematics(); o.refresh()
    want = acc + kp * (target - st["q"]) + kd * (vt - st["qdot"])
    w.step_n(1); o.step(1)
    got = (w.download(F.JOINT_VELOCITY) - st["qdot"]) * 500.0
    assert np.abs(got[:, 1:] - want[:, 1:]).max() / np.abs(want[:, 1:]).max() < 2e-3
    assert rel(w.download(F.JOINT_VELOCITY), o.get("qdot", L)) < 2e-5
    assert rel(w.download(F.ACTUATOR_EFFORT)[:, 1:], o.get("actuator_applied", L)[:, 1:]) < 1e-4
    w.step_n(19); o.step(19)
    assert rel(w.download(F.JOINT_POSITION), o.get("q", L)) < 1e-4 and w.download(F.ENV_STATUS).max() == 0
    w.destroy()
    # floating base, contacts, force limits
    E, L = 48, 13
    blob = T.quadruped(0).blob()
    w = nuka.World.create_from_template(device, blob, E, control_mode=3)
    o = oracle.World(blob, E)
    o.set_control_mode(3)
    st = T.quadruped_state(E, 6)
    limit = np.full((E, L), 20.0, np.float32)
    kp, kd = np.full((E, L), 400.0, np.float32), np.full((E, L), 40.0, np.float32)
    for field, name, value in ((F.JOINT_POSITION, "q", st["q"]), (F.BASE_POSE, "base_pose", st["base_pose"]),
                               (F.DRIVE_FORCE_LIMIT, "drive_force_limit", limit), (F.DRIVE_STIFFNESS, "drive_stiffness", kp),
                               (F.DRIVE_DAMPING, "drive_damping", kd)):
        w.upload(field, value); o.set(name, value.reshape(E, -1))
    w.forward_kinematics(); o.refresh()
    w.step_n(1); o.step(1)
    # the command goes through M^-1 and the inverse of its actuated block (condition number 7e3 each way): two fp32
    # evaluations agree to 1e-4 here where the plain PD step agrees to 2e-5
    assert rel(w.download(F.JOINT_VELOCITY), o.get("qdot", L)) < 3e-4
    w.step_n(39); o.step(39)
    assert rel(w.download(F.JOINT_POSITION), o.get("q", L)) < 1e-3 and rel(w.download(F.BASE_POSE), o.get("base_pose", 7)) < 1e-3
    assert w.download(F.ENV_STATUS).max() == 0
    assert w.download(F.BASE_POSE)[:, 2].min() > 0.1                   # the controller keeps the trunks off the ground
    w.destroy()


def test_joint_limit_multipliers_carry_over(device, oracle):
    """A random fixed-base arm that runs into its joint limits: the multipliers of the limit rows persist from step to
    step (the next step's rows start from them), are readable as JOINT_LIMIT_IMPULSE, and a reset clears them."""
    import sys
    sys.path.insert(0, GOLDEN)
    import ref_cases
    E = 64
    tb = ref_cases.random_robot(1)
    L = len(tb.links)
    st = ref_cases.random_robot_state(1, E)
    w, o = make_pair(device, oracle, tb, E, {"q": st["q"], "qdot": st["qdot"]})
    seen = False
    for _ in range(6):
        w.step_n(10); o.step(10)
        mine, want = w.download(F.JOINT_LIMIT_IMPULSE).reshape(E, 2 * L), o.get("limit_multiplier", 2 * L)
        seen |= bool((want != 0).any())
        assert rel(mine, want) < 1e-2
        assert rel(w.download(F.JOINT_POSITION), o.get("q", L)) < 1e-4
    assert seen                                   # the case does reach its limits
    w.reset()
    assert not w.download(F.JOINT_LIMIT_IMPULSE).any()
    w.destroy()


def test_cylinder_manifolds_match_the_oracle(device, oracle):
    """Free cylinders and spheres over a plane (cylinder-plane with cap, rim and side contacts, cylinder-sphere in both
    slot orders, the mirrored ones in a second small scene).  One collide pass on the seeded poses, lowered so that most shapes touch: pair lists and contact counts
    bit-exact, points, normals and depths within 1e-5.  Then 30 steps: counts equal and poses within 1e-4."""
    import sys
    sys.path.insert(0, GOLDEN)
    import ref_cases
    E = 128
    tb = ref_cases.cylinder_field()
    B = len(tb.bodies)
    pose = ref_cases.cylinder_field_state(E)["body_pose"].reshape(E, B, 7).copy()
    kinds = tb.arrays()["shape_kind"]
    lowered = pose.copy()
    lowered[:, kinds == 7, 2] -= 0.08          # cylinders into the ground by up to their radius
    lowered[:, kinds == 0, 2] = 0.16           # spheres down onto them
    w, o = make_pair(device, oracle, tb, E, {"body_pose": lowered.reshape(E, -1)})
    S = w.info.contact_slots_per_env
    w.run_stage(2); o.collide()
    pc = w.download(F.PAIR_COUNT)
    assert np.array_equal(pc, o.get("pair_count", 1))
    live = np.arange(S)[None, :] < pc
    gp = w.download(F.CANDIDATE_PAIRS).reshape(E, S, 2)
    assert np.array_equal(gp[live], o.get("candidate_pairs", 2 * S).reshape(E, S, 2)[live])
    cc = w.download(F.CONTACT_COUNT)
    assert np.array_equal(cc[live], o.get("contact_count", S)[live])
    points = (np.arange(4)[None, None, :] < cc[:, :, None]) & live[:, :, None]
    seen = set()
    for env, slot in zip(*np.nonzero((cc > 0) & live)):
        seen.add((int(kinds[gp[env, slot, 0]]), int(kinds[gp[env, slot, 1]]), int(cc[env, slot])))
    assert {(7, 3, 1), (7, 3, 2), (7, 3, 4), (7, 0, 1)} <= seen
    for field, name in ((F.CONTACT_POINT, "contact_point"), (F.CONTACT_NORMAL, "contact_normal")):
        assert np.abs(w.download(field).reshape(E, S, 4, 3)[points] - o.get(name, 12 * S).reshape(E, S, 4, 3)[points]).max() < 1e-5
    assert np.abs(w.download(F.CONTACT_DEPTH).reshape(E, S, 4)[points] - o.get("contact_depth", 4 * S).reshape(E, S, 4)[points]).max() < 1e-5
    w.destroy()
    w, o = make_pair(device, oracle, tb, E, {"body_pose": pose.reshape(E, -1)})
    w.step_n(30); o.step(30)
    assert np.array_equal(w.download(F.CONTACT_COUNT), o.get("contact_count", S))
    assert rel(w.download(F.RIGID_BODY_TRANSFORM), o.get("body_pose", 7 * B)) < 1e-4
    w.destroy()
    # the mirrored slot orders: plane first, then spheres, then cylinders
    from nuka.templates import CYLINDER, SPHERE, TemplateBuilder
    mb = TemplateBuilder(dt=1 / 250.0, vel_iters=8, max_contacts=12)
    mb.add_plane(0.0, mu=0.9, contype=2, conaffinity=1)
    for k in range(2):
        mb.add_free_body((SPHERE, 0.05), 0.5, (0.0005,) * 3, (0.3 * k, 0.0, 0.15, 1, 0, 0, 0), mu=0.6, contype=1, conaffinity=7)
    for k in range(2):
        mb.add_free_body((CYLINDER, 0.08, 0.03), 0.7, (0.0013, 0.0013, 0.0022), (0.3 * k, 0.0, 0.02, 1, 0, 0, 0), mu=0.7, contype=4, conaffinity=2)
    rng = np.random.Generator(np.random.PCG64(11))
    mp = np.tile(mb.arrays()["body_pose0"].reshape(1, 5, 7), (E, 1, 1)).astype(np.float32)
    quat = rng.normal(size=(E, 2, 4)); quat /= np.linalg.norm(quat, axis=-1, keepdims=True)
    quat[: E // 4] = (1.0, 0.0, 0.0, 0.0)                       # a quarter flat on their caps
    mp[:, 3:, 3:] = quat
    mp[:, 1:3, :2] += rng.uniform(-0.08, 0.08, size=(E, 2, 2)).astype(np.float32)
    mp[:, 1:3, 2] += rng.uniform(-0.08, 0.0, size=(E, 2)).astype(np.float32)
    w, o = make_pair(device, oracle, mb, E, {"body_pose": mp.reshape(E, -1)})
    S = w.info.contact_slots_per_env
    w.run_stage(2); o.collide()
    pc = w.download(F.PAIR_COUNT)
    assert np.array_equal(pc, o.get("pair_count", 1))
    live = np.arange(S)[None, :] < pc
    gp = w.download(F.CANDIDATE_PAIRS).reshape(E, S, 2)
    cc = w.download(F.CONTACT_COUNT)
    assert np.array_equal(cc[live], o.get("contact_count", S)[live])
    points = (np.arange(4)[None, None, :] < cc[:, :, None]) & live[:, :, None]
    mk = mb.arrays()["shape_kind"]
    seen = {(int(mk[gp[env, slot, 0]]), int(mk[gp[env, slot, 1]])) for env, slot in zip(*np.nonzero((cc > 0) & live))}
    assert {(3, 7), (0, 7)} <= seen
    for field, name in ((F.CONTACT_POINT, "contact_point"), (F.CONTACT_NORMAL, "contact_normal")):
        assert np.abs(w.download(field).reshape(E, S, 4, 3)[points] - o.get(name, 12 * S).reshape(E, S, 4, 3)[points]).max() < 1e-5
    assert np.abs(w.download(F.CONTACT_DEPTH).reshape(E, S, 4)[points] - o.get("contact_depth", 4 * S).reshape(E, S, 4)[points]).max() < 1e-5
    w.destroy()


def test_operational_space_control_inputs(device, oracle):
    """Control mode 4 on the arm against the oracle with position and orientation tasks, and its input checks: a task link
    outside the articulation is refused at creation, a task link in another mode too, a non-finite target raises the
    control-failure bit of that env only and leaves its command at zero."""
    import sys
    sys.path.insert(0, GOLDEN)
    import ref_cases
    E, L = 32, 8
    tb = T.arm7(0)
    st = ref_cases.arm_osc_state(E, 0)
    with pytest.raises(nuka.NukaError) as err:
        nuka.World.create_from_template(device, tb.blob(), E, control_mode=4, osc_task_link=8)
    assert err.value.code == 1
    with pytest.raises(nuka.NukaError) as err:
        nuka.World.create_from_template(device, tb.blob(), E, control_mode=0, osc_task_link=7)
    assert err.value.code == 7
    w = nuka.World.create_from_template(device, tb.blob(), E, control_mode=4, osc_task_link=7)
    o = oracle.World(tb.blob(), E)
    o.set_control_mode(4); o.set_task_link(7)
    target = st["task_target"].copy()
    target[5, 1] = np.nan
    fields = {"q": (F.JOINT_POSITION, "q"), "qdot": (F.JOINT_VELOCITY, "qdot"), "drive_target": (F.DRIVE_TARGET, "drive_target"),
              "kp": (F.DRIVE_STIFFNESS, "drive_stiffness"), "kd": (F.DRIVE_DAMPING, "drive_damping"),
              "task_rotation": (F.TASK_ROTATION_TARGET, "task_rotation_target"), "task_frame": (F.TASK_LOCAL_POSE, "task_local_pose"),
              "null_kp": (F.TASK_NULLSPACE_STIFFNESS, "task_nullspace_stiffness"), "null_kd": (F.TASK_NULLSPACE_DAMPING, "task_nullspace_damping")}
    for key, (field, name) in fields.items():
        w.upload(field, st[key]); o.set(name, st[key].reshape(E, -1))
    w.upload(F.TASK_TARGET, target); o.set("task_target", target)
    w.forward_kinematics(); o.refresh()
    w.step_n(1); o.step(1)
    status = w.download(F.ENV_STATUS)[:, 0]
    assert status[5] == 1 << 10 and not np.delete(status, 5).any()
    assert np.array_equal(o.get("env_status", 1)[:, 0], status)
    good = np.arange(E) != 5
    assert rel(w.download(F.JOINT_VELOCITY)[good], o.get("qdot", L)[good]) < 1e-4
    w.step_n(19); o.step(19)
    # the six-row tasks amplify last-bit differences (see refparity.SENSITIVE); the position-only ones stay at 1e-5
    assert rel(w.download(F.JOINT_POSITION)[good], o.get("q", L)[good]) < 1e-3
    three_rows = good & (np.arange(E) % 2 == 1)
    assert rel(w.download(F.JOINT_POSITION)[three_rows], o.get("q", L)[three_rows]) < 1e-5
    w.reset()
    assert np.array_equal(w.download(F.TASK_LOCAL_POSE), st["task_frame"])      # task inputs survive a reset, like the drive inputs
    w.destroy()
