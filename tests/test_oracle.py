"""The CPU checker against (a) outputs of the reference's own compiled C loops
stored as golden vectors, (b) the same loops run live when the reference build
is present, (c) an independent fp64 dense recomputation, as BIDMat's own tests
do (src/test/scala/BIDMat/SMatTest.scala:42-61)."""
import os

import numpy as np
import pytest
import scipy.sparse as sp

import oracle
from util import random_csc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "spblas_ref_vectors.npz")


def golden_cases():
    z = np.load(GOLDEN)
    names = sorted({k.split("/")[0] for k in z.files})
    return z, names


@pytest.mark.parametrize("name", golden_cases()[1])
def test_oracle_matches_reference_golden_bit_exact(name):
    z, _ = golden_cases()
    g = {k.split("/")[1]: z[k] for k in z.files if k.startswith(name + "/")}
    m = int(g["m"])
    for nthreads in (1, 3, 8):
        C = oracle.dsmult(g["A"], g["data"], g["ir"], g["jc"], out=g["C0"].copy(), nthreads=nthreads)
        assert np.array_equal(C.view(np.uint32), g["C"].view(np.uint32))
        G = oracle.dsmultT(g["B"], g["data"], g["ir"], g["jc"], m, out=g["G0"].copy(), nthreads=nthreads)
        assert np.array_equal(G.view(np.uint32), g["G"].view(np.uint32))


@pytest.mark.skipif(not oracle.ref_available(), reason="reference build not present")
@pytest.mark.parametrize("k,m,n,dens", [(128, 300, 200, 0.05), (37, 100, 90, 0.2), (256, 64, 64, 0.4), (1, 50, 50, 0.3)])
def test_oracle_matches_live_reference_build(k, m, n, dens):
    rng = np.random.default_rng(k * 7 + m)
    jc, ir, data = random_csc(m, n, dens, rng, empty_cols=(1, n - 1))
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((n, k)).astype(np.float32)
    assert np.array_equal(oracle.dsmult(A, data, ir, jc), oracle.ref_smcscm(A, data, ir, jc))
    assert np.array_equal(oracle.dsmultT(B, data, ir, jc, m), oracle.ref_smcsrm(B, data, ir, jc, m))


def _dense(m, n, jc, ir, data):
    ic = oracle.uncompress_inds(jc)
    return sp.csc_matrix((data.astype(np.float64), ir, jc), shape=(m, n)), ic


@pytest.mark.parametrize("k,m,n", [(10, 30, 20), (20, 30, 10), (128, 200, 150), (257, 64, 80)])
def test_oracle_matches_fp64_dense_recomputation(k, m, n):
    """Reference-style check: compare with a dense formulation, absolute 1e-4
    (BIDMatSpec.assert_approx_eq), at the reference's shapes and beyond."""
    rng = np.random.default_rng(k + m + n)
    jc, ir, data = random_csc(m, n, 0.2, rng)
    A = rng.uniform(0, 1, (m, k)).astype(np.float32)       # `rand` operands as in the reference tests
    B = rng.uniform(0, 1, (n, k)).astype(np.float32)
    S, ic = _dense(m, n, jc, ir, data)
    C = oracle.dsmult(A, data, ir, jc)
    assert np.abs(C - (S.T @ A.astype(np.float64))).max() < 1e-4
    G = oracle.dsmultT(B, data, ir, jc, m)
    assert np.abs(G - (S @ B.astype(np.float64))).max() < 1e-4
    P = oracle.dds(A, B, ir, jc)
    Pd = np.einsum("ij,ij->i", A[ir].astype(np.float64), B[ic].astype(np.float64))
    assert np.abs(P - Pd).max() < 1e-4
    # fp64 companions agree with the dense recomputation to rounding
    C64, Cabs = oracle.dsmult_f64(A, data, ir, jc)
    assert np.allclose(C64, S.T @ A.astype(np.float64), rtol=1e-12, atol=1e-12)
    G64, _ = oracle.dsmultT_f64(B, data, ir, jc, m)
    assert np.allclose(G64, S @ B.astype(np.float64), rtol=1e-12, atol=1e-12)
    P64, Pabs = oracle.dds_f64(A, B, ir, jc)
    assert np.allclose(P64, Pd, rtol=1e-12, atol=1e-12)
    assert np.all(Cabs >= np.abs(C64) - 1e-9) and np.all(Pabs >= np.abs(P64) - 1e-9)


def test_oracle_accumulates_and_dds_stores():
    rng = np.random.default_rng(5)
    k, m, n = 16, 20, 12
    jc, ir, data = random_csc(m, n, 0.3, rng)
    A = rng.standard_normal((m, k)).astype(np.float32)
    C0 = rng.standard_normal((n, k)).astype(np.float32)
    C = oracle.dsmult(A, data, ir, jc, out=C0.copy())
    Cz = oracle.dsmult(A, data, ir, jc)
    assert np.allclose(C, C0 + Cz, atol=1e-5)


def test_oracle_thread_count_does_not_change_bits():
    rng = np.random.default_rng(9)
    k, m, n = 96, 80, 70
    jc, ir, data = random_csc(m, n, 0.25, rng)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((n, k)).astype(np.float32)
    base = (oracle.dsmult(A, data, ir, jc, nthreads=1), oracle.dsmultT(B, data, ir, jc, m, nthreads=1),
            oracle.dds(A, B, ir, jc, nthreads=1))
    for t in (2, 3, 5, 8):
        assert np.array_equal(base[0], oracle.dsmult(A, data, ir, jc, nthreads=t))
        assert np.array_equal(base[1], oracle.dsmultT(B, data, ir, jc, m, nthreads=t))
        assert np.array_equal(base[2], oracle.dds(A, B, ir, jc, nthreads=t))


def test_index_helpers_round_trip_and_check():
    rng = np.random.default_rng(2)
    m, n = 40, 25
    jc, ir, _ = random_csc(m, n, 0.2, rng, empty_cols=(0, 7, 8, 24))
    ic = oracle.uncompress_inds(jc)
    assert len(ic) == jc[-1] and np.all(np.diff(ic) >= 0)
    assert np.array_equal(oracle.compress_inds(ic, n), jc)
    assert oracle.check_csc(m, n, ir, jc) == 0
    bad = ir.copy()
    j = int(jc[1])                      # first entry of a non-empty column with >= 2 entries
    c = next(c for c in range(n) if jc[c + 1] - jc[c] >= 2)
    bad[jc[c] + 1] = bad[jc[c]]         # repeated row inside a column
    assert oracle.check_csc(m, n, bad, jc) == 3
    jcb = jc.copy(); jcb[0] = 1
    assert oracle.check_csc(m, n, ir, jcb) == 1


def test_empty_matrix_is_noop():
    k, m, n = 8, 5, 4
    jc = np.zeros(n + 1, dtype=np.int32)
    e_i = np.zeros(0, dtype=np.int32)
    e_f = np.zeros(0, dtype=np.float32)
    A = np.ones((m, k), dtype=np.float32)
    B = np.ones((n, k), dtype=np.float32)
    assert not oracle.dsmult(A, e_f, e_i, jc).any()
    assert not oracle.dsmultT(B, e_f, e_i, jc, m).any()
    assert oracle.dds(A, B, e_i, jc).shape == (0,)


@pytest.mark.skipif(not oracle.ref_available(), reason="reference build not present")
@pytest.mark.parametrize("k,m,n,dens", [(64, 120, 90, 0.1), (5, 40, 33, 0.3)])
def test_double_precision_oracle_matches_live_reference_build(k, m, n, dens):
    """dmcscm / dmcsrm (BIDMat_SPBLAS.c:294-360), bit for bit."""
    rng = np.random.default_rng(k + n)
    jc, ir, data = random_csc(m, n, dens, rng, empty_cols=(2,))
    data = data.astype(np.float64) * (1 + 1e-9)
    A = rng.standard_normal((m, k))
    B = rng.standard_normal((n, k))
    C0 = rng.standard_normal((n, k))
    G0 = rng.standard_normal((m, k))
    assert np.array_equal(oracle.dsmult_d(A, data, ir, jc, out=C0.copy(), nthreads=3),
                          oracle.ref_dmcscm(A, data, ir, jc, out=C0.copy()))
    assert np.array_equal(oracle.dsmultT_d(B, data, ir, jc, m, out=G0.copy()),
                          oracle.ref_dmcsrm(B, data, ir, jc, m, out=G0.copy()))
    ic = oracle.uncompress_inds(jc)
    assert np.allclose(oracle.dds_d(A, B, ir, jc), np.einsum("ij,ij->i", A[ir], B[ic]), rtol=1e-13, atol=1e-13)


# ---- DDS: arithmetic pinned to the reference's compiled smcscm / dmcscm loop
DDS_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "dds_ref_vectors.npz")


def dds_golden_cases():
    z = np.load(DDS_GOLDEN)
    return z, sorted({k.split("/")[0] for k in z.files})


@pytest.mark.parametrize("name", dds_golden_cases()[1])
def test_dds_oracle_matches_reference_golden_bit_exact(name):
    """The stored values were produced by the reference's own smcscm / dmcscm loop
    (one-row dense operand, column = B[:, c]; tests/golden/make_golden.py), which adds
    the products in the order DDShelper does (MatFunctions.scala:1603-1607)."""
    z, _ = dds_golden_cases()
    g = {k.split("/")[1]: z[k] for k in z.files if k.startswith(name + "/")}
    for nthreads in (1, 4):
        P = oracle.dds(g["A"], g["B"], g["ir"], g["jc"], nthreads=nthreads)
        assert np.array_equal(P.view(np.uint32), g["P"].view(np.uint32))
    P64 = oracle.dds_d(g["A"].astype(np.float64), g["B"].astype(np.float64), g["ir"], g["jc"])
    assert np.array_equal(P64.view(np.uint64), g["P64"].view(np.uint64))


@pytest.mark.skipif(not oracle.ref_available(), reason="reference build not present")
@pytest.mark.parametrize("k", [1, 7, 128, 256, 512])
def test_dds_oracle_matches_live_reference_smcscm(k):
    """smcscm with M = 1 (BIDMat_SPBLAS.c:376-388): C[0,c] = sum_j v[j]*a[ir[j]] in j
    order from a stored 0 is the dot product of DDShelper, bit for bit."""
    sys_path_golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(sys_path_golden, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    rng = np.random.default_rng(77 + k)
    m, n = 11, 9
    jc, ir, _ = random_csc(m, n, 0.5, rng, empty_cols=(4,))
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((n, k)).astype(np.float32)
    want = mg.dds_through_smcscm(A, B, ir, jc)
    got = oracle.dds(A, B, ir, jc)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    A64, B64 = rng.standard_normal((m, k)), rng.standard_normal((n, k))
    want64 = mg.dds_through_smcscm(A64, B64, ir, jc, f64=True)
    assert np.array_equal(oracle.dds_d(A64, B64, ir, jc).view(np.uint64), want64.view(np.uint64))


def test_native_build_of_the_oracle_gives_the_same_bits():
    """The -O3 -march=native build (what the benchmark times) against the plain build."""
    rng = np.random.default_rng(31)
    k, m, n = 256, 300, 120
    jc, ir, data = random_csc(m, n, 0.2, rng, empty_cols=(5,))
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((n, k)).astype(np.float32)
    C0 = rng.standard_normal((n, k)).astype(np.float32)
    try:
        oracle.use_native(False)
        plain = (oracle.dsmult(A, data, ir, jc, out=C0.copy(), nthreads=3), oracle.dsmultT(B, data, ir, jc, m, nthreads=3),
                 oracle.dds(A, B, ir, jc, nthreads=3))
        if oracle.use_native(True) != "native":
            pytest.skip("no native build on this machine")
        native = (oracle.dsmult(A, data, ir, jc, out=C0.copy(), nthreads=3), oracle.dsmultT(B, data, ir, jc, m, nthreads=3),
                  oracle.dds(A, B, ir, jc, nthreads=3))
    finally:
        oracle.use_native(False)
    for p, q in zip(plain, native):
        assert np.array_equal(p.view(np.uint32), q.view(np.uint32))
