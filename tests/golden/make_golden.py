"""Regenerates tests/golden/spblas_ref_vectors.npz.

The values come from BIDMat's own C loops smcscm / smcsrm
(jni/src/BIDMat_SPBLAS.c:364-427), compiled from a reference checkout by
oracle/build.py and called on small seeded inputs.  The reference has no
golden vectors of its own for this path (its tests are randomised
self-consistency checks), so these are outputs of the reference code itself.
DDS has no compiled twin in the reference; no DDS golden is stored.

Run from the repository root:  python tests/golden/make_golden.py [reference_root]
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from oracle import build as obuild  # noqa: E402
from util import random_csc  # noqa: E402

CASES = [
    # name, k, m, n, density, empty columns
    ("ref_shape_mult", 20, 30, 10, 0.2, ()),      # GSMatTest "matrix multiplication": bbt(20x30) * aat(30x10)
    ("ref_shape_multT", 10, 20, 30, 0.2, ()),     # GSMatTest "matrix *^": aa(10x30) *^ bb(20x30)
    ("k128_split", 128, 64, 48, 0.15, (3, 4, 47)),
    ("k130_scalar", 130, 40, 33, 0.3, (0,)),
    ("k256", 256, 50, 20, 0.5, ()),
    ("k7", 7, 25, 60, 0.1, (10, 11, 12)),
]


def main():
    if len(sys.argv) > 1:
        os.environ["BIDMAT_REFERENCE_ROOT"] = sys.argv[1]
    if not obuild.build_reference(os.environ.get("BIDMAT_REFERENCE_ROOT", obuild.DEFAULT_REFERENCE_ROOT), force=True):
        raise SystemExit("no reference checkout: cannot regenerate golden vectors")
    out = {}
    for idx, (name, k, m, n, dens, empty) in enumerate(CASES):
        rng = np.random.default_rng(1000 + idx)
        jc, ir, data = random_csc(m, n, dens, rng, empty_cols=empty)
        A = rng.standard_normal((m, k)).astype(np.float32)
        B = rng.standard_normal((n, k)).astype(np.float32)
        C0 = rng.standard_normal((n, k)).astype(np.float32)   # non-zero start: accumulate semantics
        G0 = rng.standard_normal((m, k)).astype(np.float32)
        C = oracle.ref_smcscm(A, data, ir, jc, out=C0.copy())
        G = oracle.ref_smcsrm(B, data, ir, jc, m, out=G0.copy())
        for key, val in dict(k=k, m=m, n=n, jc=jc, ir=ir, data=data, A=A, B=B, C0=C0, G0=G0, C=C, G=G).items():
            out["%s/%s" % (name, key)] = np.asarray(val)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "spblas_ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
