"""Seeded random inputs of the differential tests between the reference's own headers (oracle/_ref) and the C
restatement: analytic contact pairs and augmented-Lagrangian row laws.  Shared by tests/test_ref_differential.py and
tests/golden/make_ref_vectors.py so that the live comparison and the committed vectors see the same cases."""
import numpy as np

SPHERE, CAPSULE, BOX, PLANE, CYLINDER = 0, 1, 2, 3, 7
PAIR_KINDS = [(SPHERE, SPHERE), (SPHERE, BOX), (BOX, SPHERE), (SPHERE, PLANE), (PLANE, SPHERE), (BOX, PLANE), (PLANE, BOX),
              (BOX, BOX), (CAPSULE, PLANE), (PLANE, CAPSULE), (CAPSULE, SPHERE), (SPHERE, CAPSULE), (CAPSULE, CAPSULE),
              (CYLINDER, PLANE), (PLANE, CYLINDER), (CYLINDER, SPHERE), (SPHERE, CYLINDER)]


def _frames(quat, pos):
    """World axes of unit quaternions (wxyz), float32 arithmetic as one fixed expression, then the origin: n x 12."""
    q = quat.astype(np.float32)
    w, x, y, z = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    one, two = np.float32(1), np.float32(2)
    cx = np.stack([one - two * (y * y + z * z), two * (x * y + w * z), two * (x * z - w * y)], 1)
    cy = np.stack([two * (x * y - w * z), one - two * (x * x + z * z), two * (y * z + w * x)], 1)
    cz = np.stack([two * (x * z + w * y), two * (y * z - w * x), one - two * (x * x + y * y)], 1)
    return np.concatenate([cx, cy, cz, pos.astype(np.float32)], 1).astype(np.float32)


def _unit_quats(rng, n, snap):
    """Random orientations; a `snap` fraction is an exact multiple of 90 degrees about a coordinate axis (face ties)."""
    q = rng.normal(size=(n, 4))
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    exact = np.array([[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1],
                      [np.sqrt(0.5), np.sqrt(0.5), 0, 0], [np.sqrt(0.5), 0, np.sqrt(0.5), 0], [np.sqrt(0.5), 0, 0, np.sqrt(0.5)]])
    pick = rng.random(n) < snap
    q[pick] = exact[rng.integers(0, len(exact), pick.sum())]
    return q


def _params(rng, kind, n):
    p = np.zeros((n, 4), np.float32)
    if kind == SPHERE:
        p[:, 0] = rng.uniform(0.02, 0.4, n)
    elif kind == CAPSULE:
        p[:, 0] = rng.uniform(0.02, 0.2, n); p[:, 1] = rng.uniform(0.05, 0.5, n); p[:, 2] = p[:, 0]
    elif kind == CYLINDER:      # radius, half height; wheels (flat) and posts (long) alike
        p[:, 0] = rng.uniform(0.02, 0.3, n); p[:, 1] = rng.uniform(0.01, 0.4, n)
    elif kind == BOX:
        p[:, :3] = rng.uniform(0.02, 0.4, (n, 3))
        cube = rng.random(n) < 0.2
        p[cube, 1] = p[cube, 0]; p[cube, 2] = p[cube, 0]
    return p


def manifold_cases(ka, kb, n, seed):
    """n cases of one pair kind: frames (n x 12 each), params (n x 4 each), query radius (n).  The second shape sits
    within touching range of the first, so about half the cases are in contact; a share has axis-aligned orientations
    (box face ties, parallel capsule axes), coincident centres or equal poses on one axis."""
    rng = np.random.default_rng([seed, ka, kb])
    pa, pb = _params(rng, ka, n), _params(rng, kb, n)
    qa, qb = _unit_quats(rng, n, 0.25), _unit_quats(rng, n, 0.25)
    same = rng.random(n) < 0.15
    qb[same] = qa[same]                                   # parallel axes / aligned faces
    near = rng.random(n) < 0.1
    qb[near] = qa[near] + rng.normal(scale=1e-4, size=(near.sum(), 4))
    qb /= np.linalg.norm(qb, axis=1, keepdims=True)
    reach = np.maximum(pa[:, :3].max(1) + pa[:, 1], 0.05) + np.maximum(pb[:, :3].max(1) + pb[:, 1], 0.05)
    ta = rng.uniform(-1, 1, (n, 3))
    direction = rng.normal(size=(n, 3))
    direction /= np.linalg.norm(direction, axis=1, keepdims=True)
    axis_dir = rng.random(n) < 0.2
    direction[axis_dir] = np.eye(3)[rng.integers(0, 3, axis_dir.sum())]
    spread = 4.0 if PLANE in (ka, kb) else 1.3          # a plane is a half-space: everything below it touches
    tb = ta + direction * (reach * rng.uniform(0.0, spread, n))[:, None]
    coincide = rng.random(n) < 0.03
    tb[coincide] = ta[coincide]
    if kb == PLANE:
        qb[rng.random(n) < 0.5] = (1, 0, 0, 0)
    if ka == PLANE:
        qa[rng.random(n) < 0.5] = (1, 0, 0, 0)
    query = np.where(rng.random(n) < 0.3, 0.0, rng.uniform(0.0, 0.05, n)).astype(np.float32)
    return _frames(qa, ta), pa, _frames(qb, tb), pb, query


def run_manifolds(fn, ka, kb, cases):
    """Evaluates one binding (`orc_manifold_frames` or `ref_manifold_frames`) on the cases: counts, points, keys."""
    fa, pa, fb, pb, query = cases
    n = len(query)
    counts = np.zeros(n, np.int32)
    points = np.zeros((n, 4, 7), np.float32)
    keys = np.zeros((n, 4), np.uint64)
    for i in range(n):
        counts[i] = fn(ka, fa[i].ctypes.data, pa[i].ctypes.data, kb, fb[i].ctypes.data, pb[i].ctypes.data, float(query[i]),
                       points[i].ctypes.data, keys[i].ctypes.data)
    return counts, points, keys


LAWS = {0: (6, 2), 1: (4, 1), 2: (8, 5), 3: (12, 1), 4: (13, 4)}      # which -> (floats in, floats out)


def law_cases(which, n, seed):
    rng = np.random.default_rng([seed, 100 + which])
    sign = lambda k: rng.choice([-1.0, 1.0], k)
    mag = lambda k, lo, hi: 10.0 ** rng.uniform(lo, hi, k)
    if which == 0:      # dual rho residual compliance lower upper
        x = np.stack([sign(n) * mag(n, -4, 1), mag(n, -1, 4), sign(n) * mag(n, -6, 0), np.where(rng.random(n) < 0.5, 0.0, mag(n, -8, 0)),
                      np.zeros(n), np.zeros(n)], 1)
        kind = rng.integers(0, 4, n)
        x[:, 4] = np.select([kind == 0, kind == 1, kind == 2], [0.0, -np.inf, -mag(n, -3, 1)], -3.4028234663852886e38)
        x[:, 5] = np.select([kind == 0, kind == 1, kind == 2], [3.4028234663852886e38, 0.0, 0.0], 3.4028234663852886e38)
        x[kind == 2, 5] = -x[kind == 2, 4]
        x[rng.random(n) < 0.05, 0] = 0.0
    elif which == 1:    # dual rho mu residual
        x = np.stack([sign(n) * mag(n, -5, 1), mag(n, -1, 4), mag(n, -5, 0), sign(n) * mag(n, -7, 0)], 1)
        x[rng.random(n) < 0.1, 0] = 0.0
        x[rng.random(n) < 0.1, 2] = 1.0
    elif which == 2:    # dual_y dual_z rho res_y res_z normal mu1 mu2
        mu = mag(n, -5, 0.3)
        x = np.stack([sign(n) * mag(n, -5, 0), sign(n) * mag(n, -5, 0), mag(n, -1, 4), sign(n) * mag(n, -7, -1), sign(n) * mag(n, -7, -1),
                      mag(n, -4, 1), mu, mu], 1)
        other = rng.random(n) < 0.3
        x[other, 7] = mag(other.sum(), -5, 0.3)
        x[rng.random(n) < 0.1, 5] = 0.0                  # zero normal impulse: the cone collapses
        x[rng.random(n) < 0.05, 5] *= -1.0
        zero = rng.random(n) < 0.1
        x[zero, 0] = 0.0; x[zero, 1] = 0.0
    elif which == 3:    # point next base scale
        x = rng.normal(size=(n, 12))
        x[:, 9:] = np.where(rng.random((n, 3)) < 0.2, 0.0, mag(3 * n, -3, 2).reshape(n, 3))
    else:               # dual next last.step last.weight last.point
        x = rng.normal(size=(n, 13))
        x[:, 9] = np.where(rng.random(n) < 0.3, 0.0, rng.uniform(0.05, 1.0, n))
        again = rng.random(n) < 0.1
        x[again, 6:9] = x[again, 3:6] - x[again, 0:3]     # unchanged step: zero secant denominator
    return np.ascontiguousarray(x, dtype=np.float32)


def run_laws(fn, which, x):
    n_in, n_out = LAWS[which]
    out = np.zeros((len(x), n_out), np.float32)
    fn(which, len(x), x.ctypes.data, n_in, out.ctypes.data, n_out)
    return out


def quadruped_moving_state(env_count, seed=0):
    """Start state of the reference-GPU case with non-zero velocities: the seeded quadruped poses plus joint rates
    N(0, 0.5) rad/s and a base twist N(0, 0.3) (angular then linear, base frame), so that joint accelerations and bias forces
    are far from zero."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "nuka-physics_b200"))
    from nuka import templates as T
    st = T.quadruped_state(env_count, seed)
    rng = np.random.Generator(np.random.PCG64(7 + seed))
    qdot = np.zeros((env_count, 13), np.float32)
    qdot[:, 1:] = rng.normal(0, 0.5, size=(env_count, 12))
    twist = np.zeros((env_count, 13, 6), np.float32)
    twist[:, 0, :] = rng.normal(0, 0.3, size=(env_count, 6))
    return {"q": st["q"], "qdot": qdot, "base_pose": st["base_pose"], "link_velocity": twist.reshape(env_count, -1)}


def arm_computed_torque_state(env_count, seed=0):
    """Computed-torque case on the 7-link arm: seeded poses and joint rates, a position target near the pose, velocity and
    acceleration targets, gains kp 25 / kd 3, no force limit."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "nuka-physics_b200"))
    from nuka import templates as T
    st = T.arm7_state(env_count, seed)
    rng = np.random.Generator(np.random.PCG64(11 + seed))
    L = 8
    acc = np.zeros((env_count, L), np.float32); acc[:, 1:] = rng.normal(0, 2.0, size=(env_count, L - 1))
    target = (st["q"] + rng.normal(0, 0.2, size=(env_count, L))).astype(np.float32)
    vt = np.zeros((env_count, L), np.float32); vt[:, 1:] = rng.normal(0, 0.5, size=(env_count, L - 1))
    return {"q": st["q"], "qdot": st["qdot"], "drive_target": target, "vel_target": vt, "acc_target": acc,
            "kp": np.full((env_count, L), 25.0, np.float32), "kd": np.full((env_count, L), 3.0, np.float32)}


def quadruped_computed_torque_state(env_count, seed=0):
    """Computed-torque case on the quadruped: the seeded drop onto the feet, targets at the standing pose, gains
    kp 400 / kd 40, 20 N m force limits (the landing saturates them)."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "nuka-physics_b200"))
    from nuka import templates as T
    st = T.quadruped_state(env_count, seed)
    L = 13
    target = np.tile(T.quadruped(0).arrays()["q0"].reshape(1, L), (env_count, 1)).astype(np.float32)
    return {"q": st["q"], "base_pose": st["base_pose"], "drive_target": target,
            "kp": np.full((env_count, L), 400.0, np.float32), "kd": np.full((env_count, L), 40.0, np.float32),
            "force_limit": np.full((env_count, L), 20.0, np.float32)}


def _quat_mul(a, b):
    w1, x1, y1, z1 = a[..., 0], a[..., 1], a[..., 2], a[..., 3]
    w2, x2, y2, z2 = b[..., 0], b[..., 1], b[..., 2], b[..., 3]
    return np.stack([w1 * w2 - x1 * x2 - y1 * y2 - z1 * z2, w1 * x2 + x1 * w2 + y1 * z2 - z1 * y2,
                     w1 * y2 - x1 * z2 + y1 * w2 + z1 * x2, w1 * z2 + x1 * y2 - y1 * x2 + z1 * w2], -1)


def _quat_rot(q, v):
    qv = q[..., 1:]
    t = 2.0 * np.cross(qv, v)
    return v + q[..., :1] * t + np.cross(qv, t)


def arm_osc_state(env_count, seed=0):
    """Operational-space control (mode 4) on the 7-link arm, task link 7 with its frame 0.3 m out at the tip: world targets
    within 10 cm of the tip's start position, an orientation target within 0.3 rad of the start orientation in every
    other env (the rest track position only), task gains kp 25 / kd 10 (the task link's drive gains), posture gains
    20 / 20 towards the start pose.  (Stiffer task gains or softer posture gains and the six-row tasks of the reference's
    controller run away within a hundred steps, in its own output too.)"""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "nuka-physics_b200"))
    from nuka import templates as T
    st = T.arm7_state(env_count, seed)
    rng = np.random.Generator(np.random.PCG64(21 + seed))
    L = 8
    q = st["q"].astype(np.float64)
    pos = np.tile(np.array([0.0, 0.0, 1.0]), (env_count, 1))
    rot = np.tile(np.array([1.0, 0.0, 0.0, 0.0]), (env_count, 1))
    for i in range(7):                                       # the serial chain of templates.arm7: 0.3 m links, axes z, y, z, ...
        if i:
            pos = pos + _quat_rot(rot, np.array([0.3, 0.0, 0.0]))
        half = 0.5 * q[:, i + 1]
        axis = np.array([0.0, 0.0, 1.0]) if i % 2 == 0 else np.array([0.0, 1.0, 0.0])
        rot = _quat_mul(rot, np.concatenate([np.cos(half)[:, None], np.sin(half)[:, None] * axis[None, :]], 1))
    tip = pos + _quat_rot(rot, np.array([0.3, 0.0, 0.0]))
    target = tip + rng.uniform(-0.1, 0.1, size=(env_count, 3))
    turn = rng.normal(0, 0.15, size=(env_count, 3))
    dq = np.concatenate([np.ones((env_count, 1)), 0.5 * turn], 1)
    desired = _quat_mul(rot, dq / np.linalg.norm(dq, axis=1, keepdims=True))
    desired[1::2] = 0.0                                      # position-only tasks
    frame = np.tile(np.array([0.3, 0.0, 0.0, 1.0, 0.0, 0.0, 0.0], np.float32), (env_count, 1))
    kp = np.zeros((env_count, L), np.float32); kp[:, 7] = 25.0
    kd = np.zeros((env_count, L), np.float32); kd[:, 7] = 10.0
    return {"q": st["q"], "qdot": st["qdot"], "drive_target": st["q"].copy(), "kp": kp, "kd": kd,
            "task_target": target.astype(np.float32), "task_rotation": desired.astype(np.float32), "task_frame": frame,
            "null_kp": np.full((env_count, 1), 20.0, np.float32), "null_kd": np.full((env_count, 1), 20.0, np.float32)}


def quadruped_osc_state(env_count, seed=0):
    """Operational-space control on the landing quadruped: the first leg's foot (task link 3, frame at the foot sphere)
    reaches for a point ahead of the trunk while the other three legs, off the task chain, hold the stance through their
    own drive gains (kp 40 / kd 2); task gains 50 / 10 on link 3, posture gains 5 / 1, 20 N m force limits, an
    orientation target in every fourth env (a foot's orientation is barely reachable through three leg joints and an
    unactuated trunk: the controller saturates the limits there)."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "nuka-physics_b200"))
    from nuka import templates as T
    st = T.quadruped_state(env_count, seed)
    rng = np.random.Generator(np.random.PCG64(31 + seed))
    L = 13
    stance = np.tile(T.quadruped(0).arrays()["q0"].reshape(1, L), (env_count, 1)).astype(np.float32)
    kp = np.full((env_count, L), 40.0, np.float32); kp[:, 3] = 50.0
    kd = np.full((env_count, L), 2.0, np.float32); kd[:, 3] = 10.0
    target = st["base_pose"][:, :3].astype(np.float64) + np.array([0.24, 0.13, -0.2]) + rng.normal(0, 0.03, size=(env_count, 3))
    turn = rng.normal(0, 0.3, size=(env_count, 3))
    desired = np.concatenate([np.ones((env_count, 1)), 0.5 * turn], 1)
    desired /= np.linalg.norm(desired, axis=1, keepdims=True)
    desired[np.arange(env_count) % 4 != 0] = 0.0
    frame = np.tile(np.array([0.0, 0.0, -0.213, 1.0, 0.0, 0.0, 0.0], np.float32), (env_count, 1))
    return {"q": st["q"], "base_pose": st["base_pose"], "drive_target": stance, "kp": kp, "kd": kd,
            "force_limit": np.full((env_count, L), 20.0, np.float32),
            "task_target": target.astype(np.float32), "task_rotation": desired.astype(np.float32), "task_frame": frame,
            "null_kp": np.full((env_count, 1), 5.0, np.float32), "null_kd": np.full((env_count, 1), 1.0, np.float32)}


def quadruped_mode_state(mode, env_count, seed=0):
    """The quadruped's seeded drop under the other control modes.  1 (torque): the target field carries joint efforts,
    a feedforward effort on top.  2 (velocity): rate targets, the stiffness field is the rate gain, 15 N m force limits.
    5 (actuator): efforts inside a torque-speed envelope of 3 N m stall effort and 6 rad/s no-load speed (three times those
    efforts make the legs thrash and the trajectories chaotic within 30 steps)."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "nuka-physics_b200"))
    from nuka import templates as T
    st = T.quadruped_state(env_count, seed)
    L = 13
    rng = np.random.Generator(np.random.PCG64(3000 + 10 * mode + seed))
    out = {"q": st["q"], "base_pose": st["base_pose"]}
    joints = np.zeros((env_count, L), np.float32)
    if mode == 1:
        joints[:, 1:] = rng.normal(0, 2.0, size=(env_count, L - 1))
        out["drive_target"] = joints
        ff = np.zeros((env_count, L), np.float32)
        ff[:, 1:] = rng.normal(0, 0.5, size=(env_count, L - 1))
        out["feedforward"] = ff
    elif mode == 2:
        joints[:, 1:] = rng.normal(0, 1.0, size=(env_count, L - 1))
        out["vel_target"] = joints
        out["kp"] = np.full((env_count, L), 8.0, np.float32)
        out["force_limit"] = np.full((env_count, L), 15.0, np.float32)
    elif mode == 5:
        joints[:, 1:] = rng.normal(0, 2.0, size=(env_count, L - 1))
        out["drive_target"] = joints
        out["force_limit"] = np.full((env_count, L), 3.0, np.float32)
        out["noload_speed"] = np.full((env_count, L), 6.0, np.float32)
    else:
        raise ValueError(mode)
    return out


def cylinder_field():
    """Free cylinders and spheres over a plane, for the cylinder manifolds: six cylinders (pucks, posts, wheels on their
    side) in random orientations a few centimetres above the ground, and six spheres dropped onto and beside them.  Filters
    keep the pairs to those with an analytic manifold: cylinders meet the plane and the spheres, never each other.
    Returns the TemplateBuilder cooked through the scene round trip."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "nuka-physics_b200"))
    from nuka import templates as T
    from nuka import nks
    rng = np.random.Generator(np.random.PCG64(5000))
    tb = T.TemplateBuilder(dt=1.0 / 250.0, vel_iters=8, max_contacts=0)
    for k in range(6):
        radius, half = float(rng.uniform(0.04, 0.1)), float(rng.uniform(0.015, 0.08))
        mass = float(1200.0 * np.pi * radius * radius * 2.0 * half)
        side = mass * (3.0 * radius * radius + 4.0 * half * half) / 12.0
        tb.add_free_body((T.CYLINDER, radius, half), mass, (float(side), float(side), float(0.5 * mass * radius * radius)),
                         (0.3 * (k % 3 - 1), 0.3 * (k // 3) - 0.15, 0.14, 1.0, 0.0, 0.0, 0.0), mu=0.7, contype=4, conaffinity=2)
    for k in range(6):
        radius = float(rng.uniform(0.03, 0.06))
        mass = float(1000.0 * 4.0 / 3.0 * np.pi * radius ** 3)
        tb.add_free_body((T.SPHERE, radius), mass, (float(0.4 * mass * radius * radius),) * 3,
                         (0.3 * (k % 3 - 1), 0.3 * (k // 3) - 0.15, 0.36, 1.0, 0.0, 0.0, 0.0), mu=0.6, contype=1, conaffinity=7)
    tb.add_plane(0.0, mu=0.9, contype=2, conaffinity=1)
    return nks.cook(nks.scene_from_builder(tb), dt=1.0 / 250.0, vel_iters=8, kp=0.0, kd=0.0, scene_filters=True, ground_height=None,
                    max_contacts=48)


def cylinder_field_state(env_count, seed=0):
    """Per-env start of cylinder_field(): every cylinder in its own random orientation (a third of them exactly upright or
    exactly on their side: cap and rim contacts, and the switch between them at |axis . normal| = 0.95), the spheres
    scattered above them within a cylinder radius."""
    tb = cylinder_field()
    a = tb.arrays()
    B = len(tb.bodies)
    rng = np.random.Generator(np.random.PCG64(5001 + seed))
    pose = np.tile(a["body_pose0"].reshape(1, B, 7), (env_count, 1, 1)).astype(np.float32)
    cyl = a["shape_kind"] == 7
    sph = a["shape_kind"] == 0
    quat = rng.normal(size=(env_count, int(cyl.sum()), 4))
    quat /= np.linalg.norm(quat, axis=-1, keepdims=True)
    exact = np.array([[1.0, 0.0, 0.0, 0.0], [np.sqrt(0.5), np.sqrt(0.5), 0.0, 0.0], [np.sqrt(0.5), 0.0, np.sqrt(0.5), 0.0]])
    pick = rng.random((env_count, int(cyl.sum()))) < 0.33
    quat[pick] = exact[rng.integers(0, 3, int(pick.sum()))]
    pose[:, cyl, 3:] = quat.astype(np.float32)
    pose[:, cyl, 2] += rng.uniform(-0.02, 0.04, size=(env_count, int(cyl.sum()))).astype(np.float32)
    pose[:, sph, :2] += rng.uniform(-0.07, 0.07, size=(env_count, int(sph.sum()), 2)).astype(np.float32)
    pose[:, sph, 2] += rng.uniform(-0.05, 0.1, size=(env_count, int(sph.sum()))).astype(np.float32)
    return {"body_pose": pose.reshape(env_count, -1)}


def random_robot(seed):
    """A seeded random articulation on a ground plane, for parity runs beyond the benchmark robots: a random tree of 6 to 14
    links under a floating or a fixed base, revolute and prismatic joints with some fixed ones in between, random axes,
    offsets, masses and inertial frames, joint limits, dry friction, armature and damping on some joints, position
    actuators, spheres and boxes (or spheres and capsules: the two never mix, capsule-box pairs have no analytic manifold)
    on most links, and up to three free bodies.  Returns the TemplateBuilder."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "nuka-physics_b200"))
    from nuka import templates as T
    rng = np.random.Generator(np.random.PCG64(1000 + seed))
    floating = bool(rng.random() < 0.6)
    count = int(rng.integers(6, 15))
    round_only = bool(rng.random() < 0.5)                 # spheres + capsules, else spheres + boxes
    tb = T.TemplateBuilder(dt=1.0 / 250.0, vel_iters=6, max_contacts=0)

    def shape():
        kind = rng.random()
        if kind < 0.25:
            return None
        if kind < 0.6:
            return (T.SPHERE, float(rng.uniform(0.03, 0.07)))
        if round_only:
            return (T.CAPSULE, float(rng.uniform(0.02, 0.04)), float(rng.uniform(0.03, 0.08)))
        return (T.BOX, float(rng.uniform(0.03, 0.07)), float(rng.uniform(0.03, 0.07)), float(rng.uniform(0.03, 0.07)))

    def inertia(mass):        # of a solid box of random size: physically realisable principal moments
        return tuple(float(v) for v in T.box_inertia(mass, rng.uniform(0.06, 0.2, size=3)))

    mass = float(rng.uniform(2.0, 5.0))
    tb.add_link(None, T.FLOATING if floating else T.FIXED, mass=mass, inertia_diag=inertia(mass), shape=shape() if floating else None,
                mu=float(rng.uniform(0.5, 1.0)), contype=1, conaffinity=0, local_pos=(0.0, 0.0, 0.0) if floating else (0.0, 0.0, 0.22))
    tb.base_pose = [0.0, 0.0, 0.28, 1.0, 0.0, 0.0, 0.0]
    for i in range(1, count):
        parent = int(rng.integers(max(0, i - 4), i))
        pick = rng.random()
        jtype = T.REVOLUTE if pick < 0.65 else T.PRISMATIC if pick < 0.85 else T.FIXED
        axis = rng.normal(size=3)
        axis = tuple(float(v) for v in axis / np.linalg.norm(axis))
        mass = float(rng.uniform(0.2, 1.5))
        single = jtype != T.FIXED
        limited = single and rng.random() < 0.5
        span = 0.15 if jtype == T.PRISMATIC else 0.8
        tb.add_link(parent, jtype, axis=axis, offset=tuple(float(v) for v in rng.uniform(-0.12, 0.12, size=3)), mass=mass,
                    inertia_diag=inertia(mass), com=tuple(float(v) for v in rng.uniform(-0.04, 0.04, size=3)),
                    q0=float(rng.uniform(-0.1, 0.1)) if single else 0.0,
                    kp=float(rng.uniform(20.0, 80.0)) if single and rng.random() < 0.8 else 0.0, kd=float(rng.uniform(0.5, 2.0)) if single else 0.0,
                    force_limit=float(rng.uniform(5.0, 30.0)) if single and rng.random() < 0.3 else 0.0,
                    damping=float(rng.uniform(0.0, 0.3)) if single else 0.0, armature=float(rng.uniform(0.0, 0.02)) if single else 0.0,
                    frictionloss=float(rng.uniform(0.05, 0.4)) if single and rng.random() < 0.4 else 0.0,
                    limits=(-span * float(rng.uniform(0.3, 1.0)), span * float(rng.uniform(0.3, 1.0))) if limited else None,
                    shape=shape(), shape_pos=tuple(float(v) for v in rng.uniform(-0.03, 0.03, size=3)), mu=float(rng.uniform(0.5, 1.0)),
                    contype=1, conaffinity=0)
    for l in tb.links:                                    # a drive needs both gains for the scene's actuator record
        if l["kp"] == 0.0:
            l["kd"] = 0.0
    for k in range(int(rng.integers(0, 4))):
        if round_only:
            body = (T.SPHERE, float(rng.uniform(0.04, 0.08)))
        else:
            body = (T.BOX, float(rng.uniform(0.04, 0.08)), float(rng.uniform(0.04, 0.08)), float(rng.uniform(0.04, 0.08)))
        m = float(rng.uniform(0.2, 1.0))
        tb.add_free_body(body, m, inertia(m), (float(rng.uniform(-0.5, 0.5)), float(rng.uniform(-0.5, 0.5)), float(rng.uniform(0.09, 0.2)), 1.0, 0.0, 0.0, 0.0),
                         mu=float(rng.uniform(0.5, 1.0)), contype=1, conaffinity=3)
    tb.add_plane(0.0, mu=0.9, contype=2, conaffinity=1)
    # through the scene writer and the cooker: links come back in the tree's pre-order, the order every consumer of the
    # scene file sees
    from nuka import nks
    cooked = nks.cook(nks.scene_from_builder(tb), dt=1.0 / 250.0, vel_iters=6, kp=0.0, kd=0.0, scene_filters=True, ground_height=None,
                      max_contacts=64)
    return cooked


def random_robot_state(seed, env_count):
    """Per-env start state of random_robot(seed): joint positions near the initial ones, joint rates, a tilted base."""
    tb = random_robot(seed)
    L = len(tb.links)
    rng = np.random.Generator(np.random.PCG64(2000 + seed))
    q0 = np.array([l["q0"] for l in tb.links], np.float32)
    q = np.tile(q0, (env_count, 1)) + rng.normal(0, 0.05, size=(env_count, L)).astype(np.float32)
    qdot = rng.normal(0, 0.3, size=(env_count, L)).astype(np.float32)
    for i, l in enumerate(tb.links):
        if l["jtype"] not in (0, 1):
            q[:, i] = 0.0; qdot[:, i] = 0.0
    base = np.tile(np.array(tb.base_pose, np.float32), (env_count, 1))
    tilt = rng.normal(0, 0.15, size=(env_count, 3))
    quat = np.concatenate([np.ones((env_count, 1)), 0.5 * tilt], axis=1)
    base[:, 3:] = (quat / np.linalg.norm(quat, axis=1, keepdims=True)).astype(np.float32)
    base[:, 2] += rng.uniform(-0.03, 0.1, size=env_count).astype(np.float32)
    out = {"q": q.astype(np.float32), "qdot": qdot.astype(np.float32)}
    if tb.links[0]["jtype"] == 3:
        out["base_pose"] = base
    return out
