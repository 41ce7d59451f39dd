"""Pins of the CPU oracle (not gpu): known-answer cases taken from the reference's own tests and
independent physics identities.  The oracle is the checker of the CUDA path, so it is pinned first.

Sources of the known answers:
  reference tests/collision/test_analytical_manifold.cpp:138-361 (penetration, normal, point count of the
  analytic pairs; the positions asserted there predate the current mid-surface placement and are not used),
  tests/collision/test_lbvh_vs_sap_pair_set.cpp (pair set equals the brute-force O(n^2) set),
  tests/scenario/pairdriven_solve.cpp (momentum exchange, box resting on ground, two runs byte-identical),
  tests/scenario/free_rigid_dynamics.cpp:764-838 (rotated-gravity covariance).
"""
import ctypes
import math

import numpy as np
import pytest

from nuka import templates as T

SPHERE, CAPSULE, BOX, PLANE = 0, 1, 2, 3
IDENT = (1.0, 0.0, 0.0, 0.0)


def manifold(orc, ka, pa, qa, sa, kb, pb, qb, sb, query=0.0):
    lib = orc.lib()
    lib.orc_manifold.restype = ctypes.c_int
    f = lambda v: np.ascontiguousarray(v, dtype=np.float32)
    pose_a, pose_b = f(list(pa) + list(qa)), f(list(pb) + list(qb))
    par_a, par_b = f(list(sa) + [0.0] * (4 - len(sa))), f(list(sb) + [0.0] * (4 - len(sb)))
    out = np.zeros(28, np.float32)
    n = lib.orc_manifold(ctypes.c_uint32(ka), pose_a.ctypes.data_as(ctypes.c_void_p), par_a.ctypes.data_as(ctypes.c_void_p),
                         ctypes.c_uint32(kb), pose_b.ctypes.data_as(ctypes.c_void_p), par_b.ctypes.data_as(ctypes.c_void_p),
                         ctypes.c_float(query), out.ctypes.data_as(ctypes.c_void_p))
    return out.reshape(4, 7)[:n]


def quat_axis_angle(axis, angle):
    a = np.asarray(axis, float) / np.linalg.norm(axis)
    return (math.cos(angle / 2), *(a * math.sin(angle / 2)))


def test_sphere_sphere(oracle):
    m = manifold(oracle, SPHERE, (0, 0, 0), IDENT, (1.0,), SPHERE, (1.5, 0, 0), IDENT, (1.0,))
    assert len(m) == 1
    assert m[0, 6] == pytest.approx(0.5, abs=1e-5)
    assert np.allclose(m[0, 3:6], (-1, 0, 0), atol=1e-5)


def test_sphere_box_and_flip(oracle):
    m = manifold(oracle, SPHERE, (0, 1.5, 0), IDENT, (0.6,), BOX, (0, 0, 0), IDENT, (1, 1, 1))
    assert len(m) == 1 and m[0, 6] == pytest.approx(0.1, abs=1e-5)
    assert np.allclose(m[0, 3:6], (0, 1, 0), atol=1e-5)
    m = manifold(oracle, BOX, (0, 0, 0), IDENT, (1, 1, 1), SPHERE, (0, 1.5, 0), IDENT, (0.6,))
    assert np.allclose(m[0, 3:6], (0, -1, 0), atol=1e-5)
    # inside the box: deepest axis wins (reference case box he (1,2,3) at (4,-2,1), sphere r 0.2 at local (-0.8,0.3,0.4))
    m = manifold(oracle, SPHERE, (3.2, -1.7, 1.4), IDENT, (0.2,), BOX, (4, -2, 1), IDENT, (1, 2, 3))
    assert m[0, 6] == pytest.approx(0.4, abs=1e-5) and np.allclose(m[0, 3:6], (-1, 0, 0), atol=1e-5)


def test_sphere_plane(oracle):
    m = manifold(oracle, SPHERE, (0, 0, 0.8), IDENT, (1.0,), PLANE, (0, 0, 0), IDENT, ())
    assert len(m) == 1 and m[0, 6] == pytest.approx(0.2, abs=1e-5)
    assert np.allclose(m[0, 3:6], (0, 0, 1), atol=1e-6)


def test_box_plane_four_corners_and_flip(oracle):
    m = manifold(oracle, BOX, (0, 0, 0.9), IDENT, (1, 1, 1), PLANE, (0, 0, 0), IDENT, ())
    assert len(m) == 4
    assert np.allclose(m[:, 6], 0.1, atol=1e-5) and np.allclose(m[:, 3:6], (0, 0, 1))
    assert {(round(float(x)), round(float(y))) for x, y in m[:, :2]} == {(-1, -1), (1, -1), (-1, 1), (1, 1)}
    m = manifold(oracle, PLANE, (0, 0, 0), IDENT, (), BOX, (0, 0, 0.9), IDENT, (1, 1, 1))
    assert len(m) == 4 and np.allclose(m[:, 3:6], (0, 0, -1))


def test_box_box_face_patch_and_clip(oracle):
    m = manifold(oracle, BOX, (0, 0, 0), IDENT, (1, 1, 1), BOX, (0, 1.9, 0), IDENT, (1, 1, 1))
    assert len(m) == 4 and np.allclose(m[:, 6], 0.1, atol=1e-5) and np.allclose(m[:, 3:6], (0, -1, 0), atol=1e-5)
    assert np.allclose(m[:, 1], 0.95, atol=1e-5)
    assert {(round(float(x)), round(float(z))) for x, z in m[:, [0, 2]]} == {(-1, -1), (1, -1), (-1, 1), (1, 1)}
    m = manifold(oracle, BOX, (0, 0, 0), IDENT, (1, 1, 1), BOX, (0.5, 1.9, 0), IDENT, (1, 1, 1))
    assert len(m) == 4 and m[:, 0].min() >= -0.5 - 1e-5 and m[:, 0].max() <= 1.0 + 1e-5
    # separated boxes: no contact
    assert len(manifold(oracle, BOX, (0, 0, 0), IDENT, (1, 1, 1), BOX, (0, 2.5, 0), IDENT, (1, 1, 1))) == 0


def test_box_box_rotated_octagon_spreads(oracle):
    q = quat_axis_angle((0, 1, 0), math.pi / 4)
    m = manifold(oracle, BOX, (0, 0, 0), IDENT, (1, 1, 1), BOX, (0, 1.9, 0), q, (1, 1, 1))
    assert len(m) == 4 and np.allclose(m[:, 6], 0.1, atol=1e-4)
    assert (m[:, 0] > 0.2).any() and (m[:, 0] < -0.2).any() and (m[:, 2] > 0.2).any() and (m[:, 2] < -0.2).any()


def test_capsule_pairs(oracle):
    lay = quat_axis_angle((0, 1, 0), math.pi / 2)
    m = manifold(oracle, CAPSULE, (0, 0, 0.4), lay, (0.5, 1.0), PLANE, (0, 0, 0), IDENT, ())
    assert len(m) == 2 and np.allclose(m[:, 6], 0.1, atol=1e-5) and np.allclose(m[:, 3:6], (0, 0, 1), atol=1e-6)
    assert sorted(round(float(x)) for x in m[:, 0]) == [-1, 1]
    m = manifold(oracle, CAPSULE, (0, 0, 0), IDENT, (0.5, 1.0), SPHERE, (0.8, 0, 0), IDENT, (0.5,))
    assert len(m) == 1 and m[0, 6] == pytest.approx(0.2, abs=1e-5) and np.allclose(m[0, 3:6], (-1, 0, 0), atol=1e-5)
    # parallel capsules 0.95 apart, radii 0.5: overlap 0.05; far apart: none
    m = manifold(oracle, CAPSULE, (0, 0, 0), IDENT, (0.5, 1.0), CAPSULE, (0.95, 0, 0), IDENT, (0.5, 1.0))
    assert len(m) == 1 and m[0, 6] == pytest.approx(0.05, abs=1e-5)
    assert len(manifold(oracle, CAPSULE, (0, 0, 0), IDENT, (0.5, 1.0), CAPSULE, (3, 0, 0), IDENT, (0.5, 1.0))) == 0


def _arm_world(orc, E=4, seed=0):
    tb = T.arm7(seed)
    w = orc.World(tb.blob(), E)
    st = T.arm7_state(E, seed)
    w.set("q", st["q"]); w.set("qdot", st["qdot"]); w.refresh()
    return tb, w, st


def test_mass_matrix_is_spd_and_matches_inverse_dynamics(oracle):
    """M qdd + bias = tau: with tau = 0 the solved acceleration must satisfy M qdd = -bias."""
    tb, w, st = _arm_world(oracle)
    w.dynamics(False)
    M = w.get("mass_matrix", 49).reshape(-1, 7, 7).astype(np.float64)
    bias = w.get("bias", 7).astype(np.float64)
    qdd = w.get("qddot", 8)[:, 1:].astype(np.float64)
    assert np.abs(M - M.transpose(0, 2, 1)).max() == 0.0
    assert np.linalg.eigvalsh(M).min() > 0.0
    assert np.allclose(np.einsum("eij,ej->ei", M, qdd), -bias, rtol=2e-4, atol=2e-4)


def test_mass_matrix_equals_kinetic_energy_hessian(oracle):
    """0.5 qd^T M qd must equal the sum of link kinetic energies computed from link spatial velocities."""
    tb, w, st = _arm_world(oracle)
    w.dynamics(False)
    M = w.get("mass_matrix", 49).reshape(-1, 7, 7).astype(np.float64)
    qd = st["qdot"][:, 1:].astype(np.float64)
    v = w.get("link_velocity", 48).reshape(-1, 8, 6).astype(np.float64)
    I = tb.arrays()["inertia"].reshape(8, 6, 6).astype(np.float64)
    ke_links = 0.5 * np.einsum("eli,lij,elj->e", v, I, v)
    ke_joint = 0.5 * np.einsum("ei,eij,ej->e", qd, M, qd)
    assert np.allclose(ke_links, ke_joint, rtol=1e-5)


def test_arm_energy_is_conserved_at_small_dt(oracle):
    tb = T.arm7(0, dt=1.0 / 4000.0)
    w = oracle.World(tb.blob(), 4)
    st = T.arm7_state(4, 0)
    w.set("q", st["q"]); w.set("qdot", st["qdot"]); w.refresh()
    masses = tb.arrays()["inertia"].reshape(8, 6, 6)[:, 3, 3].astype(np.float64)

    def energy():
        w.dynamics(False)
        M = w.get("mass_matrix", 49).reshape(-1, 7, 7).astype(np.float64)
        qd = w.get("qdot", 8)[:, 1:].astype(np.float64)
        pose = w.get("link_pose", 56).reshape(-1, 8, 7).astype(np.float64)
        qw, qx, qy, qz = pose[..., 3], pose[..., 4], pose[..., 5], pose[..., 6]
        com_z = pose[..., 2] + 2.0 * (qx * qz - qw * qy) * 0.15
        return 0.5 * np.einsum("ei,eij,ej->e", qd, M, qd) + (masses * 9.81 * com_z).sum(axis=1)

    e0 = energy()
    w.step(400)
    assert np.abs(energy() - e0).max() / np.abs(e0).max() < 2e-3


def _free_box_world(orc, poses, vels=None, E=1, gravity=(0, 0, -9.81), plane=True, dt=1 / 240.0, iters=32):
    tb = T.TemplateBuilder(dt=dt, vel_iters=iters, gravity=gravity, max_contacts=8)
    for p in poses:
        tb.add_free_body((T.BOX, 0.1, 0.1, 0.1), 1.0, T.box_inertia(1.0, (0.2, 0.2, 0.2)), p, mu=0.5)
    if plane:
        tb.add_plane(0.0, mu=0.5)
    w = orc.World(tb.blob(), E)
    if vels is not None:
        w.set("body_linear_velocity", np.tile(np.asarray(vels, np.float32).reshape(1, -1), (E, 1)))
    return tb, w


def test_free_box_rests_on_ground(oracle):
    tb, w = _free_box_world(oracle, [(0, 0, 0.1005, 1, 0, 0, 0)])
    w.step(240)
    pose = w.get("body_pose", 14)[0, :7]
    vel = w.get("body_linear_velocity", 6)[0, :3]
    assert abs(pose[2] - 0.1005) < 2e-3 and np.abs(vel).max() < 1e-2 and w.get("env_status", 1)[0, 0] == 0


def test_two_free_boxes_exchange_momentum(oracle):
    tb, w = _free_box_world(oracle, [(-0.15, 0, 0, 1, 0, 0, 0), (0.15, 0, 0, 1, 0, 0, 0)], vels=[1, 0, 0, -1, 0, 0],
                            gravity=(0, 0, 0), plane=False)
    w.step(60)
    v = w.get("body_linear_velocity", 6)[0].reshape(2, 3)
    assert abs(v[:, 0].sum()) < 1e-4          # total momentum kept (equal masses)
    assert v[0, 0] <= 1e-3 and v[1, 0] >= -1e-3   # the approach is stopped (inelastic contact)
    p = w.get("body_pose", 14)[0].reshape(2, 7)
    assert p[1, 0] - p[0, 0] >= 0.2 - 2e-3      # no interpenetration beyond the slop


def test_two_runs_are_byte_identical(oracle):
    outs = []
    for _ in range(2):
        tb = T.quadruped()
        w = oracle.World(tb.blob(), 3)
        st = T.quadruped_state(3)
        w.set("q", st["q"]); w.set("base_pose", st["base_pose"]); w.refresh()
        w.step(30, threads=2)
        outs.append((w.get("q", 13).tobytes(), w.get("base_pose", 7).tobytes(), w.get("qdot", 13).tobytes()))
    assert outs[0] == outs[1]


def test_pair_set_equals_brute_force(oracle):
    """Candidate pairs == every (i<j) with overlapping AABBs, not both static, filter-admitted, not excluded."""
    E = 5
    tb = T.box_pile(0, count=20)
    tb.cfg["max_contacts"] = 256
    w = oracle.World(tb.blob(), E)
    st = T.box_pile_state(E, 0, count=20)
    st["body_pose"][:, :20, 2] *= 0.35       # squash the lattice so that many boxes overlap
    w.set("body_pose", st["body_pose"].reshape(E, -1)); w.refresh()
    w.collide()
    lo, hi = w.get("aabb_lo", 63).reshape(E, 21, 3), w.get("aabb_hi", 63).reshape(E, 21, 3)
    count, pairs = w.get("pair_count", 1)[:, 0], w.get("candidate_pairs", 512).reshape(E, 256, 2)
    a = tb.arrays()
    for e in range(E):
        expect = []
        for i in range(21):
            for j in range(i + 1, 21):
                if (hi[e, i] < lo[e, j]).any() or (lo[e, i] > hi[e, j]).any():
                    continue
                if a["body_id"][i] < 0 and a["body_id"][j] < 0:
                    continue
                if ((a["contype"][i] & a["conaffinity"][j]) | (a["contype"][j] & a["conaffinity"][i])) == 0:
                    continue
                expect.append((i, j))
        got = [tuple(p) for p in pairs[e, :count[e]]]
        assert got == expect and len(expect) > 20


def test_rotated_gravity_covariance(oracle):
    """Rotating gravity and the initial pose together rotates the trajectory (free_rigid_dynamics.cpp:764-838)."""
    q = np.array(quat_axis_angle((1, 0, 0), 0.7), np.float32)
    R = np.array([[1, 0, 0], [0, math.cos(0.7), -math.sin(0.7)], [0, math.sin(0.7), math.cos(0.7)]])
    results = []
    for rotated in (False, True):
        g = (0, 0, -9.81) if not rotated else tuple(R @ np.array([0, 0, -9.81]))
        tb = T.quadruped()
        tb.cfg["gravity"] = g
        tb.cfg["max_contacts"] = 0
        tb.bodies = [b for b in tb.bodies if b["kind"] != T.PLANE]
        w = oracle.World(tb.blob(), 1)
        st = T.quadruped_state(1)
        base = st["base_pose"].copy()
        if rotated:
            base[0, :3] = R @ base[0, :3]
            base[0, 3:] = q
        w.set("q", st["q"]); w.set("base_pose", base); w.refresh()
        w.step(40)
        results.append((w.get("base_pose", 7)[0], w.get("q", 13)[0]))
    (p0, q0), (p1, q1) = results
    assert np.allclose(R @ p0[:3].astype(np.float64), p1[:3], atol=2e-5)
    assert np.allclose(q0, q1, atol=2e-5)


# ---- row laws and contact identity: the expectations of tests/math/test_contact_tangent.cpp and
# ---- tests/constraint/test_contact_identity.cpp of the reference, evaluated on the oracle's restatements

def _law(oracle, which, values):
    import ctypes
    lib = oracle.lib()
    lib.orc_law_kat.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_double)]
    lib.orc_law_kat.restype = None
    arr = (ctypes.c_float * max(len(values), 1))(*values)
    out = (ctypes.c_double * 8)()
    lib.orc_law_kat(which, arr, out)
    return list(out)


def test_momentum_restart_signs(oracle):
    # test_contact_tangent.cpp:8-18
    scale = [2.0, 4.0, 0.0]
    assert _law(oracle, 0, [1.0, 2.0, 0.0, 0.8, 1.8, 0.0, 1.1, 2.1, 0.0] + scale)[0] < 0.0
    assert _law(oracle, 0, [0.4, 1.4, 0.0, 0.5, 1.5, 0.0, 0.8, 1.8, 0.0] + scale)[0] > 0.0
    assert _law(oracle, 0, [1.0, 2.0, 3.0, 1.0, 2.0, 3.0, 0.0, 0.0, 0.0] + scale)[0] == 0.0


def test_relaxation_finds_the_linear_root(oracle):
    # test_contact_tangent.cpp:20-35
    for beta in (0.0, 0.5):
        x, y, z, weight = _law(oracle, 1, [beta])[:4]
        assert x == 10.0 and abs(y) <= 5.0e-7 and z == 0.0
        assert abs(weight - 1.0 / 3.0) <= 1.0e-7
        assert y * y + z * z <= x * x


def test_collapsed_friction_sets_have_zero_response(oracle):
    # test_contact_tangent.cpp:37-63 (EvaluateTangentImpulse leg): zero normal impulse -> no tangent response
    for mu in (1.1e-5, 0.5, 2.0):
        for value in (0.0, 0.1):
            assert _law(oracle, 2, [10.0, 0.0, value, -value, 0.0, mu])[:5] == [0.0] * 5


def test_friction_magnitude_and_coulomb_limit(oracle):
    # test_contact_tangent.cpp:65-90 (EvaluateTangentImpulse leg)
    for mu in (1.1e-5, 0.5, 2.0):
        normal, rho = 0.05, 10.0
        radius = np.float32(mu) * np.float32(normal)
        for fraction in (0.25, 2.0):
            residual = [0.0, 0.6 * fraction * radius / rho, 0.8 * fraction * radius / rho]
            magnitude = radius * min(fraction, 1.0)
            iy, iz, yy, zz, yz = _law(oracle, 2, [rho] + residual + [normal, mu])[:5]
            assert abs(iy - 0.6 * magnitude) <= radius * 2.0e-6 and abs(iz - 0.8 * magnitude) <= radius * 2.0e-6
            if fraction < 1.0:
                assert abs(yy - rho) <= 2.0e-5 and abs(zz - rho) <= 2.0e-5


def test_contact_identity_rules(oracle):
    # test_contact_identity.cpp:47-66: stable features override point motion; without features the quantised
    # local points decide (1/4096 bins)
    import ctypes
    lib = oracle.lib()
    lib.orc_contact_identity.argtypes = [ctypes.c_uint32, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float), ctypes.c_uint32]
    lib.orc_contact_identity.restype = ctypes.c_uint64

    def ident(feature, a, b, slot=2):
        return lib.orc_contact_identity(feature, (ctypes.c_float * 3)(*a), (ctypes.c_float * 3)(*b), slot)

    a, b = (0.1, -0.2, 0.3), (-0.4, 0.5, -0.6)
    assert ident(7, a, b) == ident(7, (2.0, 3.0, 4.0), (-2.0, -3.0, -4.0))
    none = 0xffffffff
    assert ident(none, a, b) == ident(none, (0.1 + 0.00001, -0.2, 0.3), b)
    assert ident(none, a, b) != ident(none, (0.1 + 0.001, -0.2, 0.3), b)
    assert ident(7, a, b, 2) != ident(7, a, b, 3) and ident(7, a, b) != ident(8, a, b)
