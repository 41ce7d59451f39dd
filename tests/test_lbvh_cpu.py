"""The oracle's LBVH broadphase (not gpu): its pair set equals the brute-force O(n^2) set and the all-pairs route, on
the case shapes of the reference's tests/collision/test_lbvh_vs_sap_pair_set.cpp (three boxes, a plane with a box,
random boxes; two runs byte-identical) and tests/collision/test_lbvh_batched.cu (each env of a batch = that env alone)."""
import ctypes

import numpy as np
import pytest

from nuka import templates as T


def tree_pairs(orc, lo, hi):
    lo, hi = np.ascontiguousarray(lo, np.float32), np.ascontiguousarray(hi, np.float32)
    n = len(lo)
    out = np.zeros(n * (n - 1) // 2 + 1, np.uint64)
    count = orc.lib().orc_lbvh_pair_set(n, lo.ctypes.data, hi.ctypes.data, out.ctypes.data, len(out))
    return [(int(k >> np.uint64(32)), int(k & np.uint64(0xffffffff))) for k in out[:count]]


def brute_pairs(lo, hi):
    n = len(lo)
    return [(i, j) for i in range(n) for j in range(i + 1, n) if not ((hi[i] < lo[j]).any() or (lo[i] > hi[j]).any())]


def test_three_boxes_and_plane_with_box(oracle):
    lo = np.array([[0, 0, 0], [0.5, 0.5, 0.5], [5, 5, 5]], np.float32)
    hi = lo + 1.0
    assert tree_pairs(oracle, lo, hi) == [(0, 1)]
    big = np.float32(np.finfo(np.float32).max)
    lo = np.array([[-big, -big, -big], [0, 0, 0.1]], np.float32)
    hi = np.array([[big, big, big], [1, 1, 1.1]], np.float32)
    assert tree_pairs(oracle, lo, hi) == [(0, 1)]
    assert tree_pairs(oracle, lo[:1], hi[:1]) == []


@pytest.mark.parametrize("n,seed", [(2, 0), (3, 1), (17, 2), (64, 3), (257, 4), (1000, 5)])
def test_random_boxes_match_brute_force(oracle, n, seed):
    rng = np.random.default_rng(seed)
    centre = rng.uniform(-1.0, 1.0, (n, 3)).astype(np.float32)
    half = rng.uniform(0.01, 0.5 / n ** (1 / 3) + 0.05, (n, 3)).astype(np.float32)
    if n >= 17:                       # duplicate centres (equal Morton codes take the index tie-break) and one unbounded box
        centre[5] = centre[3]; centre[7] = centre[3]
        half[9] = 3.0e38
    lo, hi = centre - half, centre + half
    got = tree_pairs(oracle, lo, hi)
    assert got == brute_pairs(lo, hi) and (n < 17 or len(got) > n)
    assert tree_pairs(oracle, lo, hi) == got                     # a second run gives the same list


def test_tree_route_equals_all_pairs_route_in_a_stepped_world(oracle):
    """Both routes feed the same filters (static-static, bitmask, exclusions) and give the same canonical list, env by env."""
    E = 6
    tb = T.box_pile(0, count=20)
    tb.cfg["max_contacts"] = 256
    st = T.box_pile_state(E, 0, count=20)
    st["body_pose"][:, :20, 2] *= 0.35
    lists = []
    for mode in (1, 2):
        w = oracle.World(tb.blob(), E)
        w.set_broadphase(mode)
        w.set("body_pose", st["body_pose"].reshape(E, -1)); w.refresh()
        w.collide()
        lists.append((w.get("pair_count", 1).copy(), w.get("candidate_pairs", 512).copy(), w.get("env_status", 1).copy()))
    assert np.array_equal(lists[0][0], lists[1][0]) and np.array_equal(lists[0][1], lists[1][1]) and np.array_equal(lists[0][2], lists[1][2])
    assert lists[0][0].min() > 20
    # the articulated robot with its exclusions, stepped: trajectories are identical whichever route finds the pairs
    outs = []
    for mode in (1, 2):
        w = oracle.World(T.quadruped(0, boxes=4).blob(), 3)
        w.set_broadphase(mode)
        s = T.quadruped_state(3, 1)
        w.set("q", s["q"]); w.set("base_pose", s["base_pose"]); w.refresh()
        w.step(40)
        outs.append((w.get("q", 13).tobytes(), w.get("body_pose", 18 * 7).tobytes()))
    assert outs[0] == outs[1]


def test_batched_envs_equal_independent_envs(oracle):
    E = 4
    tb = T.box_pile(1, count=12)
    tb.cfg["max_contacts"] = 128
    st = T.box_pile_state(E, 1, count=12)
    st["body_pose"][:, :12, 2] *= 0.4
    w = oracle.World(tb.blob(), E)
    w.set_broadphase(2)
    w.set("body_pose", st["body_pose"].reshape(E, -1)); w.refresh(); w.collide()
    batched = w.get("candidate_pairs", 256)
    for e in range(E):
        one = oracle.World(tb.blob(), 1)
        one.set_broadphase(2)
        one.set("body_pose", st["body_pose"][e:e + 1].reshape(1, -1)); one.refresh(); one.collide()
        assert np.array_equal(one.get("candidate_pairs", 256)[0], batched[e])
