"""Cooks the articulated part of a ``.nks`` scene (the reference's JSON scene format, src/scene/format/nks.cpp) into a
template for this library.

Covered: one tree of rigid bodies joined by revolute / prismatic / fixed joints under a free or static root, the
bodies' inertial frames, joint axes, limits, damping, armature, initial positions, and every sphere / capsule / box
collision shape with its local frame.  The frame rules are the reference's (runtime/articulation/
articulation_state.cpp:392-426): parent-to-child is parent_frame * local_pose * joint(q), with parent_frame.position
kept apart as the parent offset.  Not covered: meshes, cylinders, heightfields, sensors, materials other than the
shapes' own friction, several trees, closed loops.

Self-collision is off by default: the scene's shapes mix capsules and boxes, and capsule-box pairs need the convex
narrowphase this library does not have.  Drives hold the initial joint positions with the given gains, as the
reference's scene-derived hold drives do in its 4096-env gate.
"""
import json

import numpy as np

from . import templates as T


def _quat_to_matrix(q):
    w, x, y, z = (float(v) for v in q)
    return np.array([[1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y)],
                     [2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x)],
                     [2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)]])


def _quat_mul(a, b):
    aw, ax, ay, az = a
    bw, bx, by, bz = b
    return (aw * bw - ax * bx - ay * by - az * bz, aw * bx + ax * bw + ay * bz - az * by,
            aw * by - ax * bz + ay * bw + az * bx, aw * bz + ax * by - ay * bx + az * bw)


def _pose(record, key):
    frame = record.get(key) or {}
    return tuple(float(v) for v in frame.get("pos", (0, 0, 0))), tuple(float(v) for v in frame.get("quat", (1, 0, 0, 0)))


_JOINT_TYPES = {"revolute": T.REVOLUTE, "hinge": T.REVOLUTE, "prismatic": T.PRISMATIC, "slide": T.PRISMATIC, "fixed": T.FIXED}


def _shape_of(cs):
    kind = cs.get("type")
    if kind == "sphere":
        return (T.SPHERE, float(cs["radius"]))
    if kind == "capsule":
        return (T.CAPSULE, float(cs["radius"]), float(cs["half_height"]))
    if kind == "box":
        return (T.BOX, *(float(v) for v in cs["half_extents"]))
    if kind == "cylinder":          # flat caps along local z; analytic manifolds against planes and spheres only
        return (T.CYLINDER, float(cs["radius"]), float(cs["half_height"]))
    raise ValueError(f"collision shape type {kind!r} has no analytic manifold here")


def cook(scene, dt=1.0 / 200.0, vel_iters=4, kp=60.0, kd=2.0, ground_height=0.0, ground_mu=1.0, self_collision=False,
         max_contacts=None, max_points=None, scene_filters=False):
    """``scene`` is a parsed .nks document (dict) or a path.  Returns a TemplateBuilder.

    ``max_points`` caps the contact points per env that get solver rows (default: the bound derived from the shape
    pairs, at most 128); a smaller cap shrinks the env's shared-memory slice, and a step that exceeds it sets the
    env's head-overflow status bit and drops the excess.

    A scene may carry its own ground (a static top-level body with a plane shape) and its own position actuators
    (an ``actuator`` component beside a joint: gain, damping, force_limit); both replace the ``ground_height`` plane and
    the ``kp`` / ``kd`` defaults.  ``scene_filters`` keeps every shape's own contype / conaffinity bits instead of the
    robot-versus-ground assignment."""
    if not isinstance(scene, dict):
        with open(scene) as f:
            scene = json.load(f)
    if scene.get("nks_version") != 1:
        raise ValueError("unsupported nks_version")
    def is_ground(node):
        return node["rigid_body"].get("is_static") and not any("rigid_body" in c for c in node.get("children", [])) and \
            any(c.get("collision_shape", {}).get("type") == "plane" for c in node.get("children", []))

    tops = [n for n in scene.get("tree", []) if "rigid_body" in n]
    grounds = [n for n in tops if is_ground(n)]
    # a top-level body with child bodies roots the articulation; a lone dynamic body is a free rigid body
    roots = [n for n in tops if not is_ground(n) and (any("rigid_body" in c for c in n.get("children", [])) or n["rigid_body"].get("is_static"))]
    free = [n for n in tops if not is_ground(n) and n not in roots]
    if len(roots) > 1:
        raise ValueError("at most one articulated tree is supported")
    self_collision = self_collision or scene_filters
    tb = T.TemplateBuilder(dt=dt, vel_iters=vel_iters, max_contacts=0)
    shape_rows = []

    def add(node, parent_link):
        rb = node["rigid_body"]
        pos, quat = _pose(node, "transform")
        joint = node.get("joint")
        if parent_link is None:
            jtype = T.FIXED if rb.get("is_static") else T.FLOATING
            tb.base_pose = [*pos, *quat]
            local_pos, local_quat, offset, axis = (0.0, 0.0, 0.0), (1.0, 0.0, 0.0, 0.0), (0.0, 0.0, 0.0), (0.0, 0.0, 1.0)
            if jtype == T.FIXED:
                local_pos, local_quat = pos, quat
        else:
            if joint is None:
                joint = {"type": "fixed"}
            if joint.get("type") not in _JOINT_TYPES:
                raise ValueError(f"joint type {joint.get('type')!r} is not supported")
            jtype = _JOINT_TYPES[joint["type"]]
            (ppos, pquat), (cpos, cquat) = _pose(joint, "parent_frame"), _pose(joint, "child_frame")
            if np.abs(np.array(cpos)).max() > 0 or abs(abs(cquat[0]) - 1.0) > 1e-9:
                raise ValueError("joints with a non-identity child frame are not supported")
            rot = _quat_to_matrix(pquat)
            local_pos = tuple(rot @ np.array(pos))
            local_quat = _quat_mul(pquat, quat)
            offset = ppos
            axis = _unit_axis(joint.get("axis", (0, 0, 1)))
        ipos, iquat = _pose(rb, "inertial")
        R = _quat_to_matrix(iquat)
        inertia = R @ np.diag([float(v) for v in rb.get("inertia", (0, 0, 0))]) @ R.T
        if abs(abs(iquat[0]) - 1.0) <= 1e-12:              # principal axes along the link's: keep the three moments
            inertia = [float(v) for v in rb.get("inertia", (0, 0, 0))]
        shapes = [c["collision_shape"] for c in node.get("children", []) if "collision_shape" in c]
        first = shapes[0] if shapes else None
        single = jtype in (T.REVOLUTE, T.PRISMATIC)
        lo, hi = (float(joint.get("lower_limit", 0.0)), float(joint.get("upper_limit", 0.0))) if single else (0.0, 0.0)
        robot_bits = dict(contype=int(first.get("contype", 1)), conaffinity=int(first.get("conaffinity", 1))) if (first and self_collision) else dict(contype=1, conaffinity=0)
        act = node.get("actuator") if single else None
        if act is not None and act.get("type") != "position":
            raise ValueError("only position actuators are carried over")
        # a position actuator's gain is the drive stiffness; without an authored damping the reference uses the
        # critically damped 2 sqrt(gain) (scene_ir.hpp:335-336)
        link_kp = float(act["gain"]) if act else (kp if single else 0.0)
        link_kd = (float(act["damping"]) if "damping" in act else 2.0 * float(act["gain"]) ** 0.5) if act else (kd if single else 0.0)
        static_root = parent_link is None and jtype == T.FIXED          # a static body carries no inertia (the reference cooks zeros)
        link = tb.add_link(parent_link, jtype, axis=axis, offset=offset, mass=0.0 if static_root else float(rb.get("mass", 0.0)),
                           inertia_diag=(0.0, 0.0, 0.0) if static_root else inertia, com=ipos,
                           q0=float(joint.get("initial_position", 0.0)) if single else 0.0, kp=link_kp, kd=link_kd,
                           force_limit=float(act.get("force_limit", 0.0)) if act else 0.0,
                           frictionloss=float(joint.get("frictionloss", 0.0)) if single else 0.0,
                           damping=float(joint.get("damping", 0.0)) if single else 0.0, armature=float(joint.get("armature", 0.0)) if single else 0.0,
                           limits=(lo, hi) if single and lo < hi else None,
                           shape=_shape_of(first) if first else None,
                           shape_pos=_pose(first, "local")[0] if first else (0, 0, 0), shape_quat=_pose(first, "local")[1] if first else (1, 0, 0, 0),
                           mu=float(first.get("friction_mu", 1.0)) if first else 1.0, local_pos=local_pos, local_quat=local_quat, **robot_bits)
        # the name a caller asks for: the joint whose child this body is, else the body's (src/c_abi/world.cpp:1186-1199)
        tb.links[link]["name"] = str((node.get("joint") or {}).get("name", "") or node.get("name", ""))
        if single and float(joint.get("stiffness", 0.0)) != 0.0:
            raise ValueError("joint springs are not carried over")
        if first:
            shape_rows.append(link)
        for cs in shapes[1:]:
            bits = dict(contype=int(cs.get("contype", 1)), conaffinity=int(cs.get("conaffinity", 1))) if self_collision else dict(contype=1, conaffinity=0)
            tb.add_link_shape(link, _shape_of(cs), *_pose(cs, "local"), mu=float(cs.get("friction_mu", 1.0)), **bits)
            shape_rows.append(link)
        for child in node.get("children", []):
            if "rigid_body" in child:
                add(child, link)

    if roots:
        add(roots[0], None)
        _exclude_welded(tb)
    for node in free:       # in document order, after the articulation's rows: the collidable row order both cookers use
        rb = node["rigid_body"]
        shapes = [c["collision_shape"] for c in node.get("children", []) if "collision_shape" in c]
        if len(shapes) != 1:
            raise ValueError("a free body needs exactly one collision shape")
        cs = shapes[0]
        (pos, quat), (ipos, iquat) = _pose(node, "transform"), _pose(rb, "inertial")
        if np.abs(np.array(_pose(cs, "local")[0])).max() > 0 or np.abs(np.array(ipos)).max() > 0 or abs(abs(iquat[0]) - 1.0) > 1e-9:
            raise ValueError("free bodies with an offset shape or inertial frame are not carried over")
        bits = dict(contype=int(cs.get("contype", 1)), conaffinity=int(cs.get("conaffinity", 1)))
        tb.add_free_body(_shape_of(cs), float(rb["mass"]), [float(v) for v in rb["inertia"]], (*pos, *quat), mu=float(cs.get("friction_mu", 1.0)), **bits)
        shape_rows.append(None)
    for g in grounds:
        plane = next(c["collision_shape"] for c in g["children"] if c.get("collision_shape", {}).get("type") == "plane")
        (gpos, gquat) = _pose(g, "transform")
        if abs(abs(gquat[0]) - 1.0) > 1e-9 or np.abs(np.array(_pose(plane, "local")[0])).max() > 0:
            raise ValueError("only horizontal ground planes at the body origin are carried over")
        bits = dict(contype=int(plane.get("contype", 1)), conaffinity=int(plane.get("conaffinity", 1))) if scene_filters else {}
        tb.add_plane(gpos[2], mu=float(plane.get("friction_mu", 1.0)), **bits)
    if not grounds and ground_height is not None:
        tb.add_plane(ground_height, mu=ground_mu)
    tb.cfg["max_contacts"] = int(max_contacts) if max_contacts is not None else max(len(shape_rows), 1)
    tb.max_points = int(max_points) if max_points is not None else 0
    return tb


def cook_native(scene_text, **options):
    """The library's own cooker (csrc/nkb_scene.cpp, what nuka_world_create_from_scene runs on a ``.nks`` path): scene
    text in, cooked template bytes out.  Keyword options are the fields of nuka_b200_cook_options_t; unset fields keep the
    library's defaults (drives from the scene's actuators only, the scene's own ground and filter bits, one candidate slot
    per admissible pair)."""
    import ctypes
    from . import _abi, _check
    lib = _abi.lib()
    o = _abi.CookOptions()
    lib.nuka_b200_cook_options_defaults(ctypes.byref(o))
    for key, value in options.items():
        if not hasattr(o, key):
            raise TypeError(f"unknown cook option {key!r}")
        setattr(o, key, value)
    text = scene_text.encode() if isinstance(scene_text, str) else bytes(scene_text)
    size = ctypes.c_size_t(0)
    _check(lib.nuka_b200_scene_cook(text, len(text), ctypes.byref(o), None, 0, ctypes.byref(size)))
    out = ctypes.create_string_buffer(size.value)
    _check(lib.nuka_b200_scene_cook(text, len(text), ctypes.byref(o), out, size.value, ctypes.byref(size)))
    return out.raw[:size.value]


def _unit_axis(axis):
    """The joint axis as the reference cooks it (src/scene/cooker.cpp:680, math::Vec3::Normalized): float32 components
    over the float32 length, zero when shorter than 1e-12."""
    x, y, z = (np.float32(v) for v in axis)
    length = np.sqrt(x * x + y * y + z * z, dtype=np.float32)
    if length < np.float32(1e-12):
        return (0.0, 0.0, 0.0)
    return (float(x / length), float(y / length), float(z / length))


def _exclude_welded(tb):
    """The reference's weld rule (src/scene/cooker.cpp:505-536, MuJoCo's weldbody and filterparent): links joined by fixed
    joints form a cluster; no pair inside a cluster, and none between a cluster and the cluster of its parent link.  Without
    fixed joints this is the parent-child exclusion add_link already applies."""
    links = tb.links
    parent = [l["parent"] for l in links]

    def weld(l):
        while parent[l] != T.NOLINK and links[l]["jtype"] == T.FIXED:
            l = parent[l]
        return l

    clusters = {}
    for l in range(len(links)):
        clusters.setdefault(weld(l), []).append(l)
    pairs = set()
    for root, members in clusters.items():
        for i, a in enumerate(members):
            for b in members[i + 1:]:
                pairs.add((min(a, b), max(a, b)))
        if parent[root] == T.NOLINK:
            continue
        for other in clusters[weld(parent[root])]:
            for member in members:
                if member != other:
                    pairs.add((min(member, other), max(member, other)))
    rows = {}
    for row, b in enumerate(tb.bodies):
        if b["link"] != T.NOLINK:
            rows.setdefault(b["link"], []).append(row)
    for a, b in pairs:
        for ra in rows.get(a, []):
            for rb in rows.get(b, []):
                tb.excluded.add((min(ra, rb) << 32) | max(ra, rb))


def _frame(pos=(0.0, 0.0, 0.0), quat=(1.0, 0.0, 0.0, 0.0)):
    return {"pos": [float(v) for v in pos], "quat": [float(v) for v in quat]}


def scene_from_builder(tb):
    """The ``.nks`` document of a procedural template: one articulated tree (revolute / prismatic / fixed joints under a
    free or static root), its shapes, position actuators for the driven joints, and the ground planes.  It is the input
    both cookers read: the reference's own loader and cooker (src/scene/format/nks.cpp, src/scene/cook/
    cook_to_model.cpp) and ``cook`` above, so that the two sides are compared on one scene file."""
    names = {T.REVOLUTE: "revolute", T.PRISMATIC: "prismatic", T.FIXED: "fixed"}
    children = {i: [] for i in range(len(tb.links))}
    for i, l in enumerate(tb.links):
        if l["parent"] != T.NOLINK:
            children[l["parent"]].append(i)
    order, body_id = [], {}

    def number(i):          # body ids follow the pre-order walk of the tree, as the loader assigns them
        body_id[i] = len(order)
        order.append(i)
        for c in children[i]:
            number(c)

    if tb.links:
        number(0)
    joint_id = {}
    for i in order:
        if i != 0:
            joint_id[i] = len(joint_id)

    def shape_node(b, name):
        kind = b["kind"]
        p = b["params"]
        cs = {"type": {T.SPHERE: "sphere", T.CAPSULE: "capsule", T.BOX: "box", T.PLANE: "plane", T.CYLINDER: "cylinder"}[kind],
              "local": _frame(b.get("geom_pos", (0, 0, 0)), b.get("geom_quat", (1, 0, 0, 0))),
              "half_extents": [float(p[0]), float(p[1]), float(p[2])] if kind == T.BOX else [0.5, 0.5, 0.5],
              "radius": float(p[0]) if kind in (T.SPHERE, T.CAPSULE, T.CYLINDER) else 0.5,
              "half_height": float(p[1]) if kind in (T.CAPSULE, T.CYLINDER) else 0.5,
              "contype": int(b["contype"]), "conaffinity": int(b["conaffinity"]), "collision_group": int(b["group"]),
              "friction_mu": float(b["mu"]), "condim": 3, "margin": 0.0, "gap": 0.0}
        return {"name": name, "collision_shape": cs}

    def node(i):
        l = tb.links[i]
        root = l["parent"] == T.NOLINK
        if l["inertia_diag"] is None:
            raise ValueError("links with a rotated inertial frame are not written")
        out = {"name": f"link{i}",
               "transform": _frame(tb.base_pose[:3], tb.base_pose[3:]) if root and l["jtype"] == T.FLOATING else _frame(l["local_pos"], l["local_quat"]),
               "rigid_body": {"parent_id": 4294967295 if root else body_id[l["parent"]], "inertial": _frame(l["com"]),
                              "mass": float(l["mass"]), "inertia": [float(v) for v in l["inertia_diag"]],
                              "is_static": bool(root and l["jtype"] == T.FIXED)}}
        if not root:
            if l["jtype"] not in names:
                raise ValueError("only revolute, prismatic and fixed joints can be written")
            lim = l["limits"]
            out["joint"] = {"name": f"joint{i}", "type": names[l["jtype"]], "parent_body": body_id[l["parent"]], "child_body": body_id[i],
                            "axis": [float(v) for v in l["axis"]], "parent_frame": _frame(l["offset"]), "child_frame": _frame(),
                            "lower_limit": float(lim[0]) if lim else 0.0, "upper_limit": float(lim[1]) if lim else 0.0,
                            "has_lower_limit": lim is not None, "has_upper_limit": lim is not None,
                            "damping": float(l["damping"]), "armature": float(l["armature"]), "stiffness": 0.0,
                            "initial_position": float(l["q0"]), "frictionloss": float(l["frictionloss"])}
            if l["kp"] != 0.0 or l["kd"] != 0.0:
                out["actuator"] = {"name": f"servo{i}", "type": "position", "joint_id": joint_id[i], "gain": float(l["kp"]),
                                   "force_limit": float(l["force_limit"]), "damping": float(l["kd"])}
        kids = [shape_node(b, f"shape{k}") for k, b in enumerate(tb.bodies) if b["link"] == i and (b["contype"] or b["conaffinity"])]
        out["children"] = kids + [node(c) for c in children[i]]
        return out

    tree = [node(0)] if tb.links else []
    for k, b in enumerate(tb.bodies):
        if b["link"] != T.NOLINK:
            continue
        if b["inv_mass"] > 0.0:
            tree.append({"name": f"body{k}", "transform": _frame(b["pose"][:3], b["pose"][3:]),
                         "rigid_body": {"parent_id": 4294967295, "inertial": _frame(b["inertial_pos"], b["inertial_quat"]), "mass": 1.0 / float(b["inv_mass"]),
                                        "inertia": [1.0 / float(v) for v in b["inv_inertia"]], "is_static": False},
                         "children": [shape_node(b, "shape")]})
            continue
        if b["kind"] != T.PLANE:
            raise ValueError("static bodies other than ground planes are not written")
        tree.append({"name": f"ground{k}", "transform": _frame(b["pose"][:3], b["pose"][3:]),
                     "rigid_body": {"parent_id": 4294967295, "inertial": _frame(), "mass": 0.0, "inertia": [0.0, 0.0, 0.0], "is_static": True},
                     "children": [shape_node(b, "plane")]})
    return {"nks_version": 1, "physics_materials": {}, "render_materials": {}, "tree": tree, "sensors": [], "exclude_pairs": [], "contact_pairs": []}


def link_names(scene):
    """Names of the tree's bodies in link order (the order ``cook`` emits them)."""
    if not isinstance(scene, dict):
        with open(scene) as f:
            scene = json.load(f)
    names = []

    def walk(node):
        names.append(node.get("name", ""))
        for child in node.get("children", []):
            if "rigid_body" in child:
                walk(child)

    for root in scene.get("tree", []):
        if "rigid_body" in root:
            walk(root)
    return names


def initial_state(tb, env_count):
    """Per-env q and base pose of the template's initial configuration (what nuka_world_reset restores)."""
    a = tb.arrays()
    q = np.tile(a["q0"].reshape(1, -1), (env_count, 1)).astype(np.float32)
    base = np.tile(a["base_pose0"].reshape(1, 7), (env_count, 1)).astype(np.float32)
    return {"q": q, "base_pose": base}


def main(argv=None):
    """``python -m nuka.nks scene.nks out.nkt``: cooks a scene file into a template file for nuka_world_create_from_scene."""
    import argparse
    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("scene")
    ap.add_argument("out")
    ap.add_argument("--dt", type=float, default=1.0 / 200.0)
    ap.add_argument("--velocity-iterations", type=int, default=4)
    ap.add_argument("--kp", type=float, default=60.0)
    ap.add_argument("--kd", type=float, default=2.0)
    ap.add_argument("--ground-height", type=float, default=0.0)
    ap.add_argument("--max-points", type=int, default=None, help="contact points per env that get solver rows")
    args = ap.parse_args(argv)
    tb = cook(args.scene, dt=args.dt, vel_iters=args.velocity_iterations, kp=args.kp, kd=args.kd, ground_height=args.ground_height,
              max_points=args.max_points)
    with open(args.out, "wb") as f:
        f.write(tb.blob())
    print(f"{args.out}: {len(tb.links)} links, {len(tb.bodies)} collidable rows")


if __name__ == "__main__":
    main()
