"""Shared by the reference-parity tests: the cases the reference's own GPU implementation was run on
(tests/golden/ref_gpu_<case>.npz, written by tests/golden/make_ref_gpu_vectors.py from oracle/_ref/ref_driver), the start
state of each, and the error measures.

Both sides consume one scene file (tests/golden/scene_<scene>.nks): the reference through its loader and cooker, this
repository through nuka.nks.cook."""
import os
import sys

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)
import ref_cases  # noqa: E402

from nuka import nks, templates as T  # noqa: E402

# case -> (scene, start state, velocity-level tolerance of the first step, trajectory tolerance)
CASES = {
    "arm7": ("arm7", lambda E: T.arm7_state(E, 0)),
    "quadruped": ("quadruped", lambda E: T.quadruped_state(E, 0)),
    "quadruped_moving": ("quadruped", lambda E: ref_cases.quadruped_moving_state(E, 0)),
    "pile12": ("pile12", lambda E: {"body_pose": T.box_pile_state(E, 0, count=12)["body_pose"].reshape(E, -1)}),
    "quadbox": ("quadbox", lambda E: T.quadruped_state(E, 0)),
    "humanoid": ("humanoid", lambda E: T.humanoid_state(E, 0)),
}
# contact points per env that get solver rows, where the procedural template sets its own capacity
MAX_POINTS = {"pile12": 72, "quadbox": 40, "humanoid": 48}


def load(case):
    path = os.path.join(GOLDEN, f"ref_gpu_{case}.npz")
    if not os.path.exists(path):
        return None
    return dict(np.load(path))


def template(case, ref):
    """This library's cook of the case's scene with the run's settings; drives come from the scene's actuators."""
    E, L, n, B, S, iters = (int(v) for v in ref["run"][:6])
    scene = CASES[case][0]
    tb = nks.cook(os.path.join(GOLDEN, f"scene_{scene}.nks"), dt=float(ref["run_dt"][0]), vel_iters=iters, kp=0.0, kd=0.0,
                  scene_filters=True, ground_height=None, max_contacts=S, max_points=MAX_POINTS.get(case))
    return tb, E, L, n, S


def err_env(got, want, floor=0.0):
    """Largest per-env error: each env's max |got - want| over that env's own max |want| (not one scale for the batch);
    `floor` bounds the scale from below for quantities that can vanish."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    E = want.shape[0]
    d = np.abs(got - want).reshape(E, -1).max(axis=1)
    scale = np.maximum(np.abs(want).reshape(E, -1).max(axis=1), floor)
    return float((d / np.maximum(scale, 1e-300)).max())


def err_envs(got, want, floor=0.0):
    """Per-env errors as in err_env, one per env."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    E = want.shape[0]
    d = np.abs(got - want).reshape(E, -1).max(axis=1)
    return d / np.maximum(np.maximum(np.abs(want).reshape(E, -1).max(axis=1), floor), 1e-300)


def assert_velocity_parity(got, want, first, tag):
    """Post-solve velocities.  After one step: within 1e-5 for at least 95 % of the envs and 1e-4 for all.  The block
    descent stops at its sweep limit in envs whose feet start inside the ground, and an iteration that has not converged
    amplifies the last-bit differences between two fp32 evaluations (the reference's own GPU result and a CPU evaluation of
    the same algorithm differ by 2e-5 in 2 % of these envs, by 1e-7 in the rest).  Along a trajectory: 1e-3."""
    d = err_envs(got, want, floor=1.0)
    if first:
        assert np.percentile(d, 95) < 1e-5 and d.max() < 1e-4, (tag, float(np.percentile(d, 95)), float(d.max()))
    else:
        assert d.max() < 1e-3, (tag, float(d.max()))


def exact_acceleration(mass, bias, n):
    """-M^-1 bias solved in double precision from the reference's own fp32 mass matrix and bias: the value every fp32
    solve of that system approximates."""
    M = np.asarray(mass, np.float64).reshape(-1, n, n)
    b = np.asarray(bias, np.float64).reshape(-1, n)
    return np.linalg.solve(M, -b[..., None])[..., 0]
