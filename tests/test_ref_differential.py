"""The C restatement against the reference's OWN compiled headers (not gpu).

oracle/_ref/libref_headers.so is built by oracle/Makefile from the reference checkout (analytical_manifold.hpp,
augmented_row.hpp; nothing copied).  Both sides are compiled without floating-point contraction and fed the same
seeded inputs, so agreement is required bit for bit: contact counts, stable feature keys, and every float.  Where the
checkout is absent (another machine) the live comparison is skipped and the committed vectors
(tests/golden/ref_vectors.npz, written by tests/golden/make_ref_vectors.py from the same library) still pin the
restatement."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import ref_cases as RC

N_LIVE = 12000          # cases per pair kind / law in the live comparison
NAMES = {0: "sphere", 1: "capsule", 2: "box", 3: "plane", 7: "cylinder"}


def ulps(a, b):
    """Distance in units of the last place between two float32 arrays (0 where bit-identical, NaN matches NaN)."""
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7fffffff), ia)
    ib = np.where(ib < 0, -(ib & 0x7fffffff), ib)
    d = np.abs(ia - ib)
    return np.where(np.isnan(a) & np.isnan(b), 0, d)


@pytest.fixture(scope="module")
def strict(oracle):
    return oracle.strict_lib()


@pytest.fixture(scope="module")
def ref(oracle):
    lib = oracle.ref_lib()
    if lib is None:
        pytest.skip("reference checkout absent: the committed vectors pin the restatement instead")
    return lib


@pytest.mark.parametrize("ka,kb", RC.PAIR_KINDS, ids=[f"{NAMES[a]}-{NAMES[b]}" for a, b in RC.PAIR_KINDS])
def test_manifolds_match_the_reference_header(strict, ref, ka, kb):
    cases = RC.manifold_cases(ka, kb, N_LIVE, seed=7)
    got = RC.run_manifolds(strict.orc_manifold_frames, ka, kb, cases)
    want = RC.run_manifolds(ref.ref_manifold_frames, ka, kb, cases)
    assert (want[0] >= 0).all()
    assert np.array_equal(got[0], want[0]), "contact counts differ"
    assert 0.2 < (want[0] > 0).mean() < 0.95, "the case generator must produce both touching and separated pairs"
    assert np.array_equal(got[2], want[2]), "stable feature keys differ"
    assert ulps(got[1], want[1]).max() <= 1


@pytest.mark.parametrize("which", sorted(RC.LAWS))
def test_row_laws_match_the_reference_header(strict, ref, which):
    x = RC.law_cases(which, N_LIVE, seed=11)
    got = RC.run_laws(strict.orc_law_batch, which, x)
    want = RC.run_laws(ref.ref_law_batch, which, x)
    assert ulps(got, want).max() <= 1
    assert np.isfinite(want).mean() > 0.9


def test_committed_reference_vectors(strict):
    """The same comparison against vectors committed from the reference's library: runs on every machine."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_vectors.npz")
    z = np.load(path)
    n = int(z["n"])
    for ka, kb in RC.PAIR_KINDS:
        cases = RC.manifold_cases(ka, kb, n, seed=int(z["seed"]))
        counts, points, keys = RC.run_manifolds(strict.orc_manifold_frames, ka, kb, cases)
        tag = f"m{ka}{kb}"
        assert np.array_equal(counts, z[tag + "_count"]) and np.array_equal(keys, z[tag + "_keys"])
        assert ulps(points, z[tag + "_points"]).max() <= 1
    for which in sorted(RC.LAWS):
        x = RC.law_cases(which, n, seed=int(z["seed"]))
        assert ulps(RC.run_laws(strict.orc_law_batch, which, x), z[f"law{which}"]).max() <= 1
