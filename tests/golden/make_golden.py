"""Regenerates tests/golden/spblas_ref_vectors.npz.

The values come from BIDMat's own C loops smcscm / smcsrm
(jni/src/BIDMat_SPBLAS.c:364-427), compiled from a reference checkout by
oracle/build.py and called on small seeded inputs.  The reference has no
golden vectors of its own for this path (its tests are randomised
self-consistency checks), so these are outputs of the reference code itself.
DDS has no compiled twin in the reference, but its arithmetic does: smcscm with a
one-row dense operand computes C[0,c] = sum_j v[j] * a[ir[j]] in j order, one rounded
multiply and one rounded add per term starting from the stored 0
(BIDMat_SPBLAS.c:376-388).  With column c holding rows 0..k-1 and the values of
B[:, c], and a = A[:, r] as a 1 x k matrix, that is DDShelper's
"dsum += a(k)*b(k)" (MatFunctions.scala:1603-1607) bit for bit.  dds_ref_vectors.npz
stores DDS results obtained from the reference's loop in this way.

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


DDS_CASES = [
    # name, k, rows of S (columns of A), columns of S (columns of B), density
    ("dds_k1", 1, 9, 7, 0.5),
    ("dds_k7", 7, 12, 10, 0.4),
    ("dds_k128", 128, 20, 16, 0.3),
    ("dds_k256", 256, 24, 12, 0.3),
    ("dds_k512", 512, 10, 8, 0.4),
    ("dds_k130", 130, 15, 9, 0.3),
]


def dds_through_smcscm(A, B, ir, jc, f64=False):
    """DDS values computed by the reference's compiled smcscm / dmcscm loop: one call
    per distinct row r of the pattern, with a = A[r] as a 1 x k dense operand and a
    sparse operand whose column c holds rows 0..k-1 with the values B[c]."""
    ft = np.float64 if f64 else np.float32
    fn = oracle.ref_dmcscm if f64 else oracle.ref_smcscm
    n, k = B.shape
    sjc = (np.arange(n + 1) * k).astype(np.int32)
    sir = np.tile(np.arange(k, dtype=np.int32), n)
    sdata = np.ascontiguousarray(B, dtype=ft).reshape(-1)
    ic = oracle.uncompress_inds(jc)
    out = np.zeros(len(ir), dtype=ft)
    for r in np.unique(ir):
        a = np.ascontiguousarray(A[r], dtype=ft).reshape(k, 1)        # 1 x k, column-major
        dots = fn(a, sdata, sir, sjc).reshape(n)                      # <A[r], B[c]> for every c
        sel = ir == r
        out[sel] = dots[ic[sel]]
    return out


def make_dds(out):
    for idx, (name, k, m, n, dens) in enumerate(DDS_CASES):
        rng = np.random.default_rng(2000 + idx)
        jc, ir, _ = random_csc(m, n, dens, rng, empty_cols=(1,))
        A = rng.standard_normal((m, k)).astype(np.float32)
        B = rng.standard_normal((n, k)).astype(np.float32)
        P = dds_through_smcscm(A, B, ir, jc)
        P64 = dds_through_smcscm(A.astype(np.float64), B.astype(np.float64), ir, jc, f64=True)
        for key, val in dict(k=k, m=m, n=n, jc=jc, ir=ir, A=A, B=B, P=P, P64=P64).items():
            out["%s/%s" % (name, key)] = np.asarray(val)


def main():
    if len(sys.argv) > 1:
        os.environ["BIDMAT_REFERENCE_ROOT"] = sys.argv[1]
    if not obuild.build_reference(force=True):
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
    dds = {}
    make_dds(dds)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dds_ref_vectors.npz")
    np.savez_compressed(path, **dds)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
