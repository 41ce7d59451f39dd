"""Procedural world templates for the benchmark configurations.

The reference obtains articulated templates by cooking scene files (USD/MJCF importers that are not
available here); these builders produce the same cooked content directly: per-link tree, joint frames,
6x6 spatial inertias in the convention of the reference's ``MakeSpatialInertia``
(src/runtime/articulation/articulation_state.cpp:307-342), collidable rows with their shape table
(src/phi/backend_cuda/ops/prims_types.cuh:33-47), parent-child pair exclusions
(src/scene/cooker.cpp:470-538) and the solver configuration (src/nk/pipeline/pipeline.hpp:35-57).
All random draws use ``numpy.random.Generator(PCG64(seed))``.
"""
import math

import numpy as np

from . import nkt

REVOLUTE, PRISMATIC, FIXED, FLOATING = 0, 1, 2, 3
SPHERE, CAPSULE, BOX, PLANE, CYLINDER = 0, 1, 2, 3, 7          # the reference's collision/shape_kind.hpp:10-17
NOLINK = 0xFFFFFFFF
FLT_BIG = 3.0e38


def spatial_inertia(mass, diag, com):
    """[[Icom + m(c.c 1 - c c^T), m c^x], [-m c^x, m 1]] about the link frame, angular-first.

    ``diag`` is the rotational inertia about the centre of mass in link axes: three principal moments, or a full 3x3."""
    c = np.asarray(com, dtype=np.float64)
    I = np.zeros((6, 6))
    if mass <= 0.0:
        return I.astype(np.float32)
    diag = np.asarray(diag, dtype=np.float64)
    I[:3, :3] = (np.diag(diag) if diag.ndim == 1 else diag) + mass * (c.dot(c) * np.eye(3) - np.outer(c, c))
    cx = np.array([[0, -c[2], c[1]], [c[2], 0, -c[0]], [-c[1], c[0], 0]])
    I[:3, 3:] = mass * cx
    I[3:, :3] = -mass * cx
    I[3:, 3:] = mass * np.eye(3)
    return I.astype(np.float32)


def box_inertia(mass, size):
    sx, sy, sz = size
    return mass / 12.0 * np.array([sy * sy + sz * sz, sx * sx + sz * sz, sx * sx + sy * sy])


class TemplateBuilder:
    def __init__(self, dt, vel_iters, pos_iters=32, gravity=(0.0, 0.0, -9.81), max_contacts=0, contact_margin=0.0,
                 max_points=0):
        self.links, self.bodies, self.excluded = [], [], set()
        self.max_points = max_points    # contact points per env that get solver rows; 0 = derived bound, at most 128
        self.extra_shapes = False
        self.cfg = dict(dt=dt, gravity=gravity, vel_iters=vel_iters, pos_iters=pos_iters, pos_beta=0.3, pos_slop=0.001,
                        contact_margin=contact_margin, baumgarte_max_velocity=FLT_BIG, overlap_recovery_velocity=0.0,
                        velocity_tolerance=1.0e-5, max_contacts=max_contacts, max_pairs=0)
        self.base_pose = [0, 0, 0, 1, 0, 0, 0]

    def add_link(self, parent, jtype, axis=(0, 0, 1), offset=(0, 0, 0), mass=0.0, inertia_diag=(0, 0, 0), com=(0, 0, 0),
                 q0=0.0, kp=0.0, kd=0.0, force_limit=0.0, damping=0.0, armature=0.0, frictionloss=0.0, limits=None,
                 shape=None, shape_pos=(0, 0, 0), shape_quat=(1, 0, 0, 0), mu=1.0, contype=1, conaffinity=0,
                 local_pos=(0, 0, 0), local_quat=(1, 0, 0, 0)):
        """Adds a link and its mirrored collidable row; ``shape`` is (kind, p0, p1, p2) or None."""
        index = len(self.links)
        body = len(self.bodies)
        self.links.append(dict(parent=NOLINK if parent is None else parent, jtype=jtype, axis=axis, offset=offset, mass=mass,
                               inertia=spatial_inertia(mass, inertia_diag, com), com=com, inertia_diag=tuple(float(v) for v in inertia_diag) if np.ndim(inertia_diag) == 1 else None, q0=q0, kp=kp, kd=kd,
                               force_limit=force_limit, damping=damping, armature=armature, frictionloss=frictionloss,
                               limits=limits, body=body, geom=0 if shape is None else 1, geom_pos=shape_pos,
                               geom_quat=shape_quat, local_pos=local_pos, local_quat=local_quat))
        kind, params = (SPHERE, (0.0, 0.0, 0.0)) if shape is None else (shape[0], shape[1:])
        self.bodies.append(dict(kind=kind, params=tuple(params) + (0.0,) * (4 - len(params)),
                                contype=0 if shape is None else contype, conaffinity=0 if shape is None else conaffinity,
                                group=0, body_id=body, link=index, mu=mu, inv_mass=0.0, inv_inertia=(0, 0, 0),
                                inertial_pos=(0, 0, 0), inertial_quat=(1, 0, 0, 0), pose=(0, 0, 0, 1, 0, 0, 0),
                                geom=0 if shape is None else 1, geom_pos=tuple(shape_pos), geom_quat=tuple(shape_quat)))
        if parent is not None:
            a, b = self.links[parent]["body"], body
            self.excluded.add((min(a, b) << 32) | max(a, b))
        return index

    def add_link_shape(self, link, shape, shape_pos=(0, 0, 0), shape_quat=(1, 0, 0, 0), mu=1.0, contype=1, conaffinity=0, group=0):
        """Adds one more collidable row to ``link``.  Rows of one link, and rows of a link and its parent, never pair."""
        body = len(self.bodies)
        self.bodies.append(dict(kind=shape[0], params=tuple(shape[1:]) + (0.0,) * (5 - len(shape)), contype=contype,
                                conaffinity=conaffinity, group=group, body_id=body, link=link, mu=mu, inv_mass=0.0,
                                inv_inertia=(0, 0, 0), inertial_pos=(0, 0, 0), inertial_quat=(1, 0, 0, 0),
                                pose=(0, 0, 0, 1, 0, 0, 0), geom=1, geom_pos=tuple(shape_pos), geom_quat=tuple(shape_quat)))
        self.extra_shapes = True
        return body

    def add_free_body(self, shape, mass, inertia_diag, pose, mu=1.0, contype=1, conaffinity=1):
        body = len(self.bodies)
        self.bodies.append(dict(kind=shape[0], params=tuple(shape[1:]) + (0.0,) * (5 - len(shape)), contype=contype,
                                conaffinity=conaffinity, group=0, body_id=body, link=NOLINK, mu=mu, inv_mass=1.0 / mass,
                                inv_inertia=tuple(1.0 / np.asarray(inertia_diag, dtype=np.float64)), inertial_pos=(0, 0, 0),
                                inertial_quat=(1, 0, 0, 0), pose=tuple(pose)))
        return body

    def add_plane(self, height=0.0, mu=1.0, contype=2, conaffinity=1):
        body = len(self.bodies)
        self.bodies.append(dict(kind=PLANE, params=(0.0,) * 4, contype=contype, conaffinity=conaffinity, group=0, body_id=-1,
                                link=NOLINK, mu=mu, inv_mass=0.0, inv_inertia=(0, 0, 0), inertial_pos=(0, 0, 0),
                                inertial_quat=(1, 0, 0, 0), pose=(0, 0, height, 1, 0, 0, 0)))
        return body

    def arrays(self):
        L, B = len(self.links), len(self.bodies)
        f32, u32 = np.float32, np.uint32
        c = self.cfg

        def lf(key, width=1, default=0.0):
            return np.array([np.atleast_1d(l.get(key, default)) for l in self.links], dtype=f32).reshape(L * width)

        def bf(key, width=1):
            return np.array([np.atleast_1d(b[key]) for b in self.bodies], dtype=f32).reshape(B * width)

        limits = [l["limits"] for l in self.links]
        out = {
            "cfg_f": np.array([c["dt"], *c["gravity"], c["pos_beta"], c["pos_slop"], c["contact_margin"],
                               c["baumgarte_max_velocity"], c["overlap_recovery_velocity"], c["velocity_tolerance"]], dtype=f32),
            "cfg_u": np.array([c["vel_iters"], c["pos_iters"], c["max_contacts"], c["max_pairs"], L, B], dtype=u32),
            "parent": np.array([l["parent"] for l in self.links], dtype=u32),
            "jtype": np.array([l["jtype"] for l in self.links], dtype=u32),
            "link_body": np.array([l["body"] for l in self.links], dtype=u32),
            "geom_kind": np.array([l["geom"] for l in self.links], dtype=u32),
            "limit_flags": np.array([0 if lim is None else 3 for lim in limits], dtype=u32),
            "axis": lf("axis", 3), "local_pos": lf("local_pos", 3), "local_quat": lf("local_quat", 4),
            "parent_offset": lf("offset", 3), "com": lf("com", 3),
            "inertia": np.array([l["inertia"] for l in self.links], dtype=f32).reshape(L * 36),
            "damping": lf("damping"), "armature": lf("armature"), "frictionloss": lf("frictionloss"),
            "stiffness": np.zeros(L, f32), "spring_ref": np.zeros(L, f32),
            "limit_lower": np.array([0.0 if lim is None else lim[0] for lim in limits], dtype=f32),
            "limit_upper": np.array([0.0 if lim is None else lim[1] for lim in limits], dtype=f32),
            "geom_pos": lf("geom_pos", 3), "geom_quat": lf("geom_quat", 4),
            "q0": lf("q0"), "base_pose0": np.array(self.base_pose, dtype=f32),
            "kp0": lf("kp"), "kd0": lf("kd"), "force_limit0": lf("force_limit"),
            "shape_kind": np.array([b["kind"] for b in self.bodies], dtype=u32),
            "contype": np.array([b["contype"] for b in self.bodies], dtype=u32),
            "conaffinity": np.array([b["conaffinity"] for b in self.bodies], dtype=u32),
            "group": np.array([b["group"] for b in self.bodies], dtype=u32),
            "body_to_link": np.array([b["link"] for b in self.bodies], dtype=u32),
            "body_id": np.array([b["body_id"] for b in self.bodies], dtype=np.int32),
            "shape_params": bf("params", 4), "mu": bf("mu"), "inv_mass": bf("inv_mass"), "inv_inertia": bf("inv_inertia", 3),
            "inertial_pos": bf("inertial_pos", 3), "inertial_quat": bf("inertial_quat", 4), "body_pose0": bf("pose", 7),
        }
        excluded = set(self.excluded)
        if self.extra_shapes:
            # several rows per link: per-row shape frames, and no pairs inside a link or between a link and its parent
            out["body_geom_kind"] = np.array([b.get("geom", 0) for b in self.bodies], dtype=u32)
            out["body_geom_pos"] = np.array([b.get("geom_pos", (0, 0, 0)) for b in self.bodies], dtype=f32).reshape(B * 3)
            out["body_geom_quat"] = np.array([b.get("geom_quat", (1, 0, 0, 0)) for b in self.bodies], dtype=f32).reshape(B * 4)
            for a in range(B):
                la = self.bodies[a]["link"]
                if la == NOLINK:
                    continue
                for b in range(a + 1, B):
                    lb = self.bodies[b]["link"]
                    if lb == NOLINK:
                        continue
                    if la == lb or self.links[la]["parent"] == lb or self.links[lb]["parent"] == la:
                        excluded.add((a << 32) | b)
        out["excluded"] = np.array(sorted(excluded), dtype=np.uint64)
        if self.max_points:
            out["max_points"] = np.array([self.max_points], dtype=u32)
        names = [l.get("name", "") for l in self.links]
        if any(names):
            # NUL-terminated UTF-8 names in link order, padded to whole words: what nuka_world_get_dof_name serves
            raw = b"".join(n.encode() + b"\0" for n in names)
            out["link_names"] = np.frombuffer(raw + b"\0" * (-len(raw) % 4), dtype=u32).copy()
        return out

    def blob(self):
        return nkt.pack(self.arrays())


def dof_count(arrays):
    width = {REVOLUTE: 1, PRISMATIC: 1, FIXED: 0, FLOATING: 6}
    return int(sum(width[int(t)] for t in arrays["jtype"]))


def arm7(seed=0, dt=1.0 / 500.0):
    """Config 1: fixed root + 7 revolute links in series, 0.3 m each, axes alternating z/y, gravity only."""
    rng = np.random.Generator(np.random.PCG64(seed))
    tb = TemplateBuilder(dt=dt, vel_iters=4, max_contacts=0)
    tb.add_link(None, FIXED, local_pos=(0.0, 0.0, 1.0))
    masses = rng.uniform(0.5, 3.0, size=7)
    for i in range(7):
        tb.add_link(i, REVOLUTE, axis=(0, 0, 1) if i % 2 == 0 else (0, 1, 0), offset=(0.0 if i == 0 else 0.3, 0, 0),
                    mass=float(masses[i]), inertia_diag=box_inertia(float(masses[i]), (0.3, 0.05, 0.05)), com=(0.15, 0, 0))
    return tb


def arm7_state(env_count, seed=0):
    rng = np.random.Generator(np.random.PCG64(seed + 1))
    q = np.zeros((env_count, 8), np.float32)
    qd = np.zeros((env_count, 8), np.float32)
    q[:, 1:] = rng.uniform(-math.pi / 4, math.pi / 4, size=(env_count, 7))
    qd[:, 1:] = rng.normal(0.0, 0.1, size=(env_count, 7))
    return {"q": q, "qdot": qd}


QUAD_STANCE = (0.0, 0.8, -1.5)


def _add_quadruped(tb, kp=40.0, kd=1.0, mu=0.8):
    trunk = tb.add_link(None, FLOATING, mass=6.9, inertia_diag=box_inertia(6.9, (0.38, 0.09, 0.11)),
                        shape=(BOX, 0.19, 0.045, 0.055), mu=mu)
    for sx in (1.0, -1.0):
        for sy in (1.0, -1.0):
            hip = tb.add_link(trunk, REVOLUTE, axis=(1, 0, 0), offset=(0.19 * sx, 0.047 * sy, 0.0), mass=0.6,
                              inertia_diag=(4.0e-4, 6.0e-4, 4.0e-4), com=(0, 0, 0), q0=QUAD_STANCE[0], kp=kp, kd=kd)
            thigh = tb.add_link(hip, REVOLUTE, axis=(0, 1, 0), offset=(0.0, 0.08 * sy, 0.0), mass=1.0,
                                inertia_diag=box_inertia(1.0, (0.03, 0.03, 0.213)), com=(0, 0, -0.1065), q0=QUAD_STANCE[1],
                                kp=kp, kd=kd)
            tb.add_link(thigh, REVOLUTE, axis=(0, 1, 0), offset=(0.0, 0.0, -0.213), mass=0.2,
                        inertia_diag=box_inertia(0.2, (0.02, 0.02, 0.213)), com=(0, 0, -0.1065), q0=QUAD_STANCE[2], kp=kp, kd=kd,
                        shape=(SPHERE, 0.022), shape_pos=(0, 0, -0.213), mu=mu)
    return trunk


def quadruped(seed=0, dt=1.0 / 200.0, vel_iters=4, boxes=0):
    """Config 2 (and, with ``boxes``, config 5): floating-base quadruped on a ground plane."""
    # with boxes: 4 foot points + 4 per resting box + box-box manifolds; 40 points with solver rows cover the scenes seen
    # (mean 20), more sets the env's head-overflow status bit
    tb = TemplateBuilder(dt=dt, vel_iters=vel_iters, max_contacts=8 if boxes == 0 else 24, max_points=0 if boxes == 0 else 40)
    _add_quadruped(tb)
    tb.base_pose = [0, 0, 0.31, 1, 0, 0, 0]
    rng = np.random.Generator(np.random.PCG64(seed))
    for k in range(boxes):
        ang = 2.0 * math.pi * (k + rng.uniform(0.0, 1.0)) / max(boxes, 1)
        rad = rng.uniform(0.5, 1.0)
        tb.add_free_body((BOX, 0.05, 0.05, 0.05), 1.0, box_inertia(1.0, (0.1, 0.1, 0.1)),
                         (rad * math.cos(ang), rad * math.sin(ang), 0.05, 1, 0, 0, 0), mu=0.8, contype=1, conaffinity=1)
    tb.add_plane(0.0, mu=0.8)
    return tb


def quadruped_state(env_count, seed=0):
    rng = np.random.Generator(np.random.PCG64(seed + 1))
    q = np.zeros((env_count, 13), np.float32)
    stance = np.tile(np.array(QUAD_STANCE, np.float32), 4)
    q[:, 1:] = stance + rng.normal(0.0, 0.05, size=(env_count, 12))
    base = np.zeros((env_count, 7), np.float32)
    base[:, 2] = rng.uniform(0.28, 0.34, size=env_count)
    base[:, 3] = 1.0
    return {"q": q, "base_pose": base}


def humanoid(seed=0, dt=1.0 / 200.0, vel_iters=8, self_collision=True):
    """Config 3: floating pelvis, two 6-DoF legs (3-1-2), 3-DoF waist, two 7-DoF arms (3-1-3); capsule colliders.

    Every capsule hangs from its joint down to the next joint of its chain (short stubs where joints coincide) and
    left and right limbs share their dimensions.  All capsules collide with the ground.  Self-contact is between
    the long segments (thigh, shin, upper arm, forearm) of different limbs, selected by filter bits: the stubs of
    coincident joints and the trunk overlap their neighbours by construction and stay out of it."""
    rng = np.random.Generator(np.random.PCG64(seed))
    # 30 capsule-plane candidates are always live (the plane's box is unbounded) + 24 limb-limb pairs
    tb = TemplateBuilder(dt=dt, vel_iters=vel_iters, max_contacts=56 if self_collision else 32, max_points=48 if self_collision else 0)
    specs = []   # (name, parent_name, axis, offset, capsule?)

    def chain(prefix, parent, axes, offsets):
        prev = parent
        for i, (ax, off) in enumerate(zip(axes, offsets)):
            name = f"{prefix}{i}"
            specs.append((name, prev, ax, off))
            prev = name
        return prev

    X, Y, Z = (1, 0, 0), (0, 1, 0), (0, 0, 1)
    for side, sy in (("l", 1.0), ("r", -1.0)):
        chain(f"leg_{side}", "pelvis", [Z, X, Y, Y, Y, X],
              [(0, 0.09 * sy, -0.05), (0, 0, 0), (0, 0, 0), (0, 0, -0.38), (0, 0, -0.38), (0, 0, 0)])
    waist = chain("waist", "pelvis", [Z, X, Y], [(0, 0, 0.08), (0, 0, 0), (0, 0, 0)])
    for side, sy in (("l", 1.0), ("r", -1.0)):
        chain(f"arm_{side}", waist, [Y, X, Z, Y, Z, X, Y],
              [(0, 0.19 * sy, 0.32), (0, 0, 0), (0, 0, 0), (0, 0, -0.28), (0, 0, -0.02), (0, 0, -0.24), (0, 0, 0)])
    radii = rng.uniform(0.03, 0.07, size=len(specs) + 1)
    lengths = np.full(len(specs) + 1, 0.06)
    lengths[0] = 0.12
    for i, (name, parent, axis, offset) in enumerate(specs):
        reach = float(np.linalg.norm(offset))
        parent_row = 0 if parent == "pelvis" else [s[0] for s in specs].index(parent) + 1
        if parent != "pelvis" and parent[:5] == name[:5] and reach > 0.1:
            lengths[parent_row] = reach            # the parent's capsule spans to this joint
    for i, (name, parent, axis, offset) in enumerate(specs):     # mirror the right side onto the left
        if "_r" in name:
            twin = [s[0] for s in specs].index(name.replace("_r", "_l")) + 1
            radii[i + 1] = radii[twin]
            lengths[i + 1] = lengths[twin]
    volumes = math.pi * radii ** 2 * lengths + 4.0 / 3.0 * math.pi * radii ** 3
    masses = 35.0 * volumes / volumes.sum()
    index = {}

    limbs = {"leg_l": 0, "leg_r": 1, "arm_l": 2, "arm_r": 3}

    def capsule_link(i, parent, jtype, axis, offset, kp):
        r, ln, m = float(radii[i]), float(lengths[i]), float(masses[i])
        contype, conaffinity = 1, 0
        name = specs[i - 1][0] if i > 0 else "pelvis"
        if self_collision and ln > 0.1 and name[:5] in limbs:
            bit = 4 << limbs[name[:5]]                    # a long segment answers to every other limb's bit
            contype, conaffinity = 1 | bit, (4 | 8 | 16 | 32) & ~bit
        diag = (m * (3 * r * r + ln * ln) / 12.0, m * (3 * r * r + ln * ln) / 12.0, 0.5 * m * r * r)
        return tb.add_link(parent, jtype, axis=axis, offset=offset, mass=m, inertia_diag=diag, com=(0, 0, -0.5 * ln),
                           kp=kp, kd=0.05 * kp, shape=(CAPSULE, r, 0.5 * ln), shape_pos=(0, 0, -0.5 * ln), mu=0.8,
                           contype=contype, conaffinity=conaffinity, armature=0.01)

    index["pelvis"] = capsule_link(0, None, FLOATING, Z, (0, 0, 0), 0.0)
    for i, (name, parent, axis, offset) in enumerate(specs):
        index[name] = capsule_link(i + 1, index[parent], REVOLUTE, axis, offset, 300.0)
    tb.base_pose = [0, 0, 0.05 + 0.38 + 0.38 + 0.06 + float(radii[[s[0] for s in specs].index('leg_l5') + 1]) + 0.005, 1, 0, 0, 0]
    tb.add_plane(0.0, mu=0.8, contype=2, conaffinity=1)
    return tb


def humanoid_state(env_count, seed=0):
    rng = np.random.Generator(np.random.PCG64(seed + 1))
    q = np.zeros((env_count, 30), np.float32)
    q[:, 1:] = rng.normal(0.0, 0.1, size=(env_count, 29))
    return {"q": q}


def box_pile(seed=0, dt=1.0 / 240.0, vel_iters=8, count=48):
    """Config 4: free boxes on a 4x4x3 jittered lattice above a plane (template holds the nominal lattice)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    tb = TemplateBuilder(dt=dt, vel_iters=vel_iters, max_contacts=6 * count, max_points=6 * count)
    for k in range(count):
        he = rng.uniform(0.02, 0.1, size=3)
        rho = rng.uniform(500.0, 2000.0)
        mass = float(rho * 8.0 * he.prod())
        ix, iy, iz = k % 4, (k // 4) % 4, k // 16
        pose = ((ix - 1.5) * 0.25, (iy - 1.5) * 0.25, 0.15 + iz * 0.25, 1, 0, 0, 0)
        tb.add_free_body((BOX, *map(float, he)), mass, box_inertia(mass, 2.0 * he), pose, mu=0.8)
    tb.add_plane(0.0, mu=0.8)
    return tb


def box_pile_state(env_count, seed=0, count=48):
    rng = np.random.Generator(np.random.PCG64(seed + 1))
    tb = box_pile(seed, count=count)
    pose = np.tile(tb.arrays()["body_pose0"].reshape(1, count + 1, 7), (env_count, 1, 1)).astype(np.float32)
    pose[:, :count, :3] += rng.uniform(-0.02, 0.02, size=(env_count, count, 3))
    quat = rng.normal(size=(env_count, count, 4))
    quat /= np.linalg.norm(quat, axis=-1, keepdims=True)
    pose[:, :count, 3:] = quat
    return {"body_pose": pose}
