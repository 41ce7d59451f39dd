"""Writes tests/golden/ref_vectors.npz: outputs of the reference's own headers (oracle/_ref/libref_headers.so) on
the seeded cases of ref_cases.py.  Run where the reference checkout exists:  python tests/golden/make_ref_vectors.py"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import orc
import ref_cases as RC

N, SEED = 300, 2024


def main():
    ref = orc.ref_lib()
    if ref is None:
        raise SystemExit("no reference checkout: cannot build oracle/_ref")
    out = {"n": np.int64(N), "seed": np.int64(SEED)}
    for ka, kb in RC.PAIR_KINDS:
        counts, points, keys = RC.run_manifolds(ref.ref_manifold_frames, ka, kb, RC.manifold_cases(ka, kb, N, SEED))
        out[f"m{ka}{kb}_count"], out[f"m{ka}{kb}_points"], out[f"m{ka}{kb}_keys"] = counts, points, keys
    for which in sorted(RC.LAWS):
        out[f"law{which}"] = RC.run_laws(ref.ref_law_batch, which, RC.law_cases(which, N, SEED))
    np.savez_compressed(os.path.join(HERE, "ref_vectors.npz"), **out)


if __name__ == "__main__":
    main()
