"""The per-env tree broadphase on the GPU: the same canonical pair list as the admissible-pair table route and as the
oracle's restatement of the reference's LBVH, env by env, and identical trajectories whichever route finds the pairs
(the reference checks its tree against brute force and SAP the same way, tests/collision/test_lbvh_vs_sap_pair_set.cpp,
and batched against independent builds, tests/collision/test_lbvh_batched.cu)."""
import numpy as np
import pytest

import nuka
from nuka import Field as F, templates as T

pytestmark = pytest.mark.gpu


def pile_worlds(device, oracle, count, E, seed, squash, slots):
    tb = T.box_pile(seed, count=count)
    tb.cfg["max_contacts"] = slots
    tb.max_points = 64
    st = T.box_pile_state(E, seed, count=count)
    st["body_pose"][:, :count, 2] *= squash
    worlds = []
    for mode in (1, 2):
        w = nuka.World.create_from_template(device, tb.blob(), E)
        w.set_broadphase(mode)
        w.upload(F.RIGID_BODY_TRANSFORM, st["body_pose"]); w.forward_kinematics()
        worlds.append(w)
    o = oracle.World(tb.blob(), E)
    o.set_broadphase(2)
    o.set("body_pose", st["body_pose"].reshape(E, -1)); o.refresh()
    return worlds, o


@pytest.mark.parametrize("count,squash", [(3, 0.5), (12, 0.4), (33, 0.35), (48, 0.3), (63, 0.3)])
def test_tree_pairs_equal_table_pairs_and_the_oracle_tree(device, oracle, count, squash):
    E, S = 37, 512
    (table, tree), o = pile_worlds(device, oracle, count, E, 3, squash, S)
    table.run_stage(2); tree.run_stage(2); o.collide()
    want_count, want = o.get("pair_count", 1), o.get("candidate_pairs", 2 * S)
    for w in (table, tree):
        assert np.array_equal(w.download(F.PAIR_COUNT), want_count)
        assert np.array_equal(w.download(F.CANDIDATE_PAIRS), want)
        assert np.array_equal(w.download(F.CONTACT_COUNT), o.get("contact_count", S))
    assert want_count.min() > count // 2            # the squashed lattice really overlaps
    table.destroy(); tree.destroy()


def test_trajectories_do_not_depend_on_the_route(device):
    E = 64
    outs = []
    for mode in (1, 2):
        w = nuka.World.create_from_template(device, T.quadruped(0, boxes=4).blob(), E)
        w.set_broadphase(mode)
        st = T.quadruped_state(E, 4)
        w.upload(F.JOINT_POSITION, st["q"]); w.upload(F.BASE_POSE, st["base_pose"]); w.forward_kinematics()
        w.step_n(60)
        outs.append([w.download(f).tobytes() for f in (F.JOINT_POSITION, F.BASE_POSE, F.RIGID_BODY_TRANSFORM, F.CANDIDATE_PAIRS, F.ENV_STATUS)])
        w.destroy()
    assert outs[0] == outs[1]


def test_pair_overflow_is_flagged_on_both_routes(device):
    E = 8
    tb = T.box_pile(5, count=20)
    tb.cfg["max_contacts"] = 16                     # far fewer slots than overlapping pairs
    st = T.box_pile_state(E, 5, count=20)
    st["body_pose"][:, :20, 2] *= 0.3
    lists = []
    for mode in (1, 2):
        w = nuka.World.create_from_template(device, tb.blob(), E)
        w.set_broadphase(mode)
        w.upload(F.RIGID_BODY_TRANSFORM, st["body_pose"]); w.forward_kinematics()
        w.run_stage(2)
        assert (w.download(F.ENV_STATUS)[:, 0] & 1).all() and (w.download(F.PAIR_COUNT) == 16).all()
        lists.append(w.download(F.CANDIDATE_PAIRS).tobytes())
        w.destroy()
    assert lists[0] == lists[1]                     # both keep the lowest keys
