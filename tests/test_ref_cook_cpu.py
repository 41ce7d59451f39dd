"""This library's scene cooker against the reference's own cook of the same scene file (not gpu).

tests/golden/scene_<name>.nks are the procedural templates written out as scene files (nuka.nks.scene_from_builder);
tests/golden/ref_cook_<name>.nkt hold the tables the reference's loader + CookToModel (src/scene/format/nks.cpp,
src/scene/cook/cook_to_model.cpp) produced from them, dumped by oracle/_ref/ref_driver --cook-only
(tests/golden/make_ref_gpu_vectors.py prepare).  Topology, frames, inertias, joint parameters, drives, shapes, filters
and excluded pairs must agree, and the scene round trip must give back the procedural template."""
import os

import numpy as np
import pytest

from nuka import nks, nkt, templates as T

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
# reference ShapeType codes of the link geometry table (src/scene/scene_ir.hpp): 0 none, 1 sphere, 2 capsule, 3 box
import sys
sys.path.insert(0, GOLDEN)
import ref_cases  # noqa: E402

CASES = {"arm7": lambda: T.arm7(0), "quadruped": lambda: T.quadruped(0), "humanoid": lambda: T.humanoid(0),
         "quadbox": lambda: T.quadruped(0, boxes=4), "pile12": lambda: T.box_pile(0, count=12),
         # seeded random articulations: random trees, prismatic and fixed joints, limits, dry friction, free bodies
         **{f"random{k}": (lambda k=k: ref_cases.random_robot(k)) for k in (0, 1, 3, 7)}}


@pytest.mark.parametrize("name", sorted(CASES))
def test_cook_matches_the_reference_cook(name):
    ref = nkt.unpack(open(os.path.join(GOLDEN, f"ref_cook_{name}.nkt"), "rb").read())
    mine = nks.cook(os.path.join(GOLDEN, f"scene_{name}.nks"), kp=0.0, kd=0.0, scene_filters=True, ground_height=None).arrays()
    L = len(ref["parent_link"])
    assert ref["artic"][1] == L == mine["cfg_u"][4] and ref["artic"][0] == T.dof_count(mine)
    assert np.array_equal(ref["parent_link"], mine["parent"]) and np.array_equal(ref["joint_type"], mine["jtype"])
    exact = (("joint_axis", "axis"), ("parent_offset", "parent_offset"), ("joint_damping", "damping"), ("joint_armature", "armature"),
             ("joint_frictionloss", "frictionloss"), ("joint_limit_lower", "limit_lower"), ("joint_limit_upper", "limit_upper"),
             ("initial_q", "q0"), ("base_pose", "base_pose0"), ("hold_targets", "q0"), ("hold_stiffness", "kp0"), ("hold_damping", "kd0"),
             ("hold_force_limits", "force_limit0"))
    for theirs, ours in exact:
        assert np.array_equal(ref[theirs], mine[ours]), theirs
    # spatial inertias are assembled from the same mass, centre and principal moments: equal to rounding
    assert np.allclose(ref["link_inertia_spatial"], mine["inertia"], rtol=0, atol=1e-7)
    local = ref["link_local_pose"].reshape(L, 7)
    jointed = np.arange(L) > 0                    # the root's local pose is its world placement (base_pose above)
    assert np.array_equal(local[jointed, :3], mine["local_pos"].reshape(L, 3)[jointed])
    assert np.array_equal(local[:, 3:], mine["local_quat"].reshape(L, 4))
    assert np.array_equal(ref["joint_limit_flags"], mine["limit_flags"])
    if L:                                         # a scene without an articulation dumps no link maps
        assert np.array_equal(ref["link_body"], mine["link_body"]) and np.array_equal(ref["body_to_link"], mine["body_to_link"])
    # collidable rows: kinds, filter bits and the parameters each kind reads
    assert np.array_equal(ref["shape_kind"], mine["shape_kind"])
    assert np.array_equal(ref["shape_contype"], mine["contype"]) and np.array_equal(ref["shape_conaffinity"], mine["conaffinity"])
    assert np.array_equal(ref["shape_group"], mine["group"])
    used = {T.SPHERE: 1, T.CAPSULE: 2, T.BOX: 3, T.PLANE: 0}
    rp, mp = ref["shape_params"].reshape(-1, 4), mine["shape_params"].reshape(-1, 4)
    for row, kind in enumerate(mine["shape_kind"]):
        if mine["contype"][row] or mine["conaffinity"][row]:
            assert np.array_equal(rp[row, :used[int(kind)]], mp[row, :used[int(kind)]]), row
    # the reference also lists the pair of two static rows (a fixed root and the ground); neither side ever pairs them
    static = (mine["inv_mass"] == 0) & ((mine["body_to_link"] == T.NOLINK) | ((mine["body_to_link"] == 0) & (mine["jtype"][0] == T.FIXED if L else False)))
    theirs = np.array([p for p in ref["excluded_pairs"] if not (static[int(p) >> 32] and static[int(p) & 0xffffffff])], np.uint64)
    assert np.array_equal(theirs, mine["excluded"])
    # friction: every collidable row's coefficient is the row's material bucket in the reference
    buckets = ref["material_buckets"].reshape(-1, 22)
    for row in range(len(mine["mu"])):
        if mine["contype"][row] or mine["conaffinity"][row]:
            assert buckets[ref["body_material_bucket"][row], 2] == pytest.approx(mine["mu"][row])


@pytest.mark.parametrize("name", sorted(CASES))
def test_scene_round_trip_gives_back_the_template(name):
    tb = CASES[name]()
    doc = nks.scene_from_builder(tb)
    back = nks.cook(doc, dt=tb.cfg["dt"], vel_iters=tb.cfg["vel_iters"], kp=0.0, kd=0.0, scene_filters=True, ground_height=None,
                    max_contacts=tb.cfg["max_contacts"], max_points=tb.max_points or None).arrays()
    want = tb.arrays()
    for key in want:
        if key in ("cfg_f", "cfg_u", "body_id", "link_names") or (key == "base_pose0" and (want["jtype"].size == 0 or want["jtype"][0] != T.FLOATING)):
            continue                                  # a fixed root's placement lives in its local pose; base_pose is unused; the writer names links by index
        got, expected = np.asarray(back[key], np.float64), np.asarray(want[key], np.float64)
        if key == "armature":                         # a root has no joint to carry one
            got, expected = got[1:], expected[1:]
        assert np.allclose(got, expected, rtol=0, atol=1e-7), key
