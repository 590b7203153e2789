"""Parity of the CUDA path with the CPU checker, through the C ABI.

Tolerances (fp32 values; structure and indices are compared bit-exactly):
  A*S, DDS : |gpu - cpu| <= 1e-5 * sum|terms|
  B*^S     : |gpu - cpu| <= 1e-4 * sum|terms|
and, at the reference's own test shapes, BIDMat's absolute 1e-4
(src/test/scala/BIDMat/BIDMatSpec.scala:13-16, GSMatTest.scala:55-83).
"""
import os

import numpy as np
import pytest
import torch

import oracle
from util import RTOL_DDS, RTOL_DSMULT, RTOL_DSMULTT, assert_close_scaled, random_csc
from gpu_util import DeviceCSC, abi_dds, abi_dds0, abi_dsmult, abi_dsmultT, dev

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "spblas_ref_vectors.npz")


def check_all_ops(k, m, n, jc, ir, data, device, rng, nonzero_start=True, normal=True):
    S = DeviceCSC(m, n, jc, ir, data, device)
    mk = (lambda s: rng.standard_normal(s).astype(np.float32)) if normal else (lambda s: rng.uniform(0, 1, s).astype(np.float32))
    A, B = mk((m, k)), mk((n, k))
    C0 = mk((n, k)) if nonzero_start else np.zeros((n, k), np.float32)
    G0 = mk((m, k)) if nonzero_start else np.zeros((m, k), np.float32)
    P0 = mk((S.nnz,)) if nonzero_start else np.zeros(S.nnz, np.float32)
    dA, dB = dev(A, device), dev(B, device)

    # A*S (accumulating)
    C = abi_dsmult(dA, S, dev(C0, device)).cpu().numpy()
    Cw = oracle.dsmult(A, data, ir, jc, out=C0.copy())
    _, Cabs = oracle.dsmult_f64(A, data, ir, jc)
    assert_close_scaled(C, Cw, Cabs + np.abs(C0), RTOL_DSMULT, "A*S k=%d" % k)

    # B*^S (accumulating)
    G = abi_dsmultT(dB, S, dev(G0, device)).cpu().numpy()
    Gw = oracle.dsmultT(B, data, ir, jc, m, out=G0.copy())
    _, Gabs = oracle.dsmultT_f64(B, data, ir, jc, m)
    assert_close_scaled(G, Gw, Gabs + np.abs(G0), RTOL_DSMULTT, "B*^S k=%d" % k)

    # DDS (accumulating on the device; the CPU loop stores)
    P = abi_dds(dA, dB, S, dev(P0, device)).cpu().numpy()
    Pw = oracle.dds(A, B, ir, jc)
    _, Pabs = oracle.dds_f64(A, B, ir, jc)
    assert_close_scaled(P, Pw + P0, Pabs + np.abs(P0), RTOL_DDS, "DDS k=%d" % k)

    # DDS0 stores
    Pz = abi_dds0(dA, dB, S, dev(P0, device)).cpu().numpy()
    assert_close_scaled(Pz, Pw, Pabs, RTOL_DDS, "DDS0 k=%d" % k)
    return C, G, P


@pytest.mark.parametrize("k", [1, 3, 4, 10, 20, 31, 32, 64, 100, 127, 128, 132, 200, 256, 260, 512, 516, 640, 1024])
def test_all_ops_over_dense_heights(cuda_device, k):
    rng = np.random.default_rng(100 + k)
    m, n = 150, 97
    jc, ir, data = random_csc(m, n, 0.15, rng, empty_cols=(0, 5, 6, 96))
    check_all_ops(k, m, n, jc, ir, data, cuda_device, rng)


def test_reference_test_shapes_absolute_eps(cuda_device):
    """GSMatTest: GMat 20x30 * GSMat 30x10 and GMat 10x30 *^ GSMat 20x30,
    density 0.2, `rand` operands, absolute 1e-4 against a dense recomputation
    (GSMatTest.scala:64-83)."""
    import scipy.sparse as sp
    rng = np.random.default_rng(7)
    for (k, m, n) in ((20, 30, 10), (10, 20, 30)):
        jc, ir, data = random_csc(m, n, 0.2, rng)
        S = DeviceCSC(m, n, jc, ir, data, cuda_device)
        A = rng.uniform(0, 1, (m, k)).astype(np.float32)
        B = rng.uniform(0, 1, (n, k)).astype(np.float32)
        full = sp.csc_matrix((data.astype(np.float64), ir, jc), shape=(m, n))
        C = abi_dsmult(dev(A, cuda_device), S, torch.zeros((n, k), device=cuda_device)).cpu().numpy()
        assert np.abs(C - full.T @ A.astype(np.float64)).max() < 1e-4
        G = abi_dsmultT(dev(B, cuda_device), S, torch.zeros((m, k), device=cuda_device)).cpu().numpy()
        assert np.abs(G - full @ B.astype(np.float64)).max() < 1e-4
        P = abi_dds(dev(A, cuda_device), dev(B, cuda_device), S, torch.zeros(S.nnz, device=cuda_device)).cpu().numpy()
        Pd = np.einsum("ij,ij->i", A[ir].astype(np.float64), B[S.ic_h].astype(np.float64))
        assert np.abs(P - Pd).max() < 1e-4


@pytest.mark.parametrize("name", ["ref_shape_mult", "ref_shape_multT", "k128_split", "k130_scalar", "k256", "k7"])
def test_against_reference_golden_vectors(cuda_device, name):
    z = np.load(GOLDEN)
    g = {k.split("/")[1]: z[k] for k in z.files if k.startswith(name + "/")}
    m, n = int(g["m"]), int(g["n"])
    S = DeviceCSC(m, n, g["jc"], g["ir"], g["data"], cuda_device)
    C = abi_dsmult(dev(g["A"], cuda_device), S, dev(g["C0"], cuda_device)).cpu().numpy()
    _, Cabs = oracle.dsmult_f64(g["A"], g["data"], g["ir"], g["jc"])
    assert_close_scaled(C, g["C"], Cabs + np.abs(g["C0"]), RTOL_DSMULT, "golden A*S " + name)
    G = abi_dsmultT(dev(g["B"], cuda_device), S, dev(g["G0"], cuda_device)).cpu().numpy()
    _, Gabs = oracle.dsmultT_f64(g["B"], g["data"], g["ir"], g["jc"], m)
    assert_close_scaled(G, g["G"], Gabs + np.abs(g["G0"]), RTOL_DSMULTT, "golden B*^S " + name)
    assert np.abs(C - g["C"]).max() < 1e-4 * max(1.0, np.abs(g["C"]).max())


@pytest.mark.parametrize("chunk", [8, 32, 96])
@pytest.mark.parametrize("k", [8, 64, 128, 256, 700])
def test_runs_crossing_chunk_boundaries(cuda_device, k, chunk, monkeypatch):
    """Tiny chunks force every column (and every row of the transposed
    product) to be split over several workers and summed by the fix-up pass."""
    monkeypatch.setenv("BIDMAT_B200_CHUNK", str(chunk))
    rng = np.random.default_rng(k + chunk)
    m, n = 60, 40
    jc, ir, data = random_csc(m, n, 0.5, rng, empty_cols=(3,))
    check_all_ops(k, m, n, jc, ir, data, cuda_device, rng)


@pytest.mark.parametrize("cols_per_block", [1, 4, 16])
@pytest.mark.parametrize("k", [12, 128, 256])
def test_transposed_product_with_column_blocks(cuda_device, k, cols_per_block, monkeypatch):
    """B*^S orders the nonzeros by (column block, row) when B is much larger
    than L2 and runs the blocks one after the other; tiny forced blocks and
    chunks exercise the slicing, the masking of the row bits and the fix-up
    across block-local chunks."""
    monkeypatch.setenv("BIDMAT_B200_COLBLOCK_COLS", str(cols_per_block))
    monkeypatch.setenv("BIDMAT_B200_CHUNK", "32")
    rng = np.random.default_rng(1000 * k + cols_per_block)
    m, n = 300, 70
    jc, ir, data = random_csc(m, n, 0.3, rng, empty_cols=(0, 1, 2, 3, 40, 69))
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    B = rng.standard_normal((n, k)).astype(np.float32)
    G0 = rng.standard_normal((m, k)).astype(np.float32)
    G = abi_dsmultT(dev(B, cuda_device), S, dev(G0, cuda_device)).cpu().numpy()
    Gw = oracle.dsmultT(B, data, ir, jc, m, out=G0.copy())
    _, Gabs = oracle.dsmultT_f64(B, data, ir, jc, m)
    assert_close_scaled(G, Gw, Gabs + np.abs(G0), RTOL_DSMULTT, "blocked B*^S")
    G2 = abi_dsmultT(dev(B, cuda_device), S, dev(G0, cuda_device)).cpu().numpy()
    assert np.array_equal(G.view(np.uint32), G2.view(np.uint32))


def test_transposed_product_with_many_rows_needs_more_sort_passes(cuda_device):
    """Row indices up to 2^21 and beyond: three and four 8-bit sort passes."""
    rng = np.random.default_rng(77)
    k = 8
    for m in (70_000, 2_200_000, 17_000_000):
        n = 50
        nnz_per_col = 40
        jc = np.arange(0, (n + 1) * nnz_per_col, nnz_per_col, dtype=np.int32)
        ir = np.concatenate([np.sort(rng.choice(m, nnz_per_col, replace=False)) for _ in range(n)]).astype(np.int32)
        ir[-1] = m - 1
        ir[-nnz_per_col:] = np.sort(ir[-nnz_per_col:])
        data = rng.uniform(0.1, 1, len(ir)).astype(np.float32)
        S = DeviceCSC(m, n, jc, ir, data, cuda_device)
        B = rng.standard_normal((n, k)).astype(np.float32)
        G = abi_dsmultT(dev(B, cuda_device), S, torch.zeros((m, k), device=cuda_device))
        rows = np.unique(ir)
        Gs = G[torch.from_numpy(rows).long().to(cuda_device)].cpu().numpy()
        want = np.zeros((m if m < 100_000 else 0, k), np.float32)
        # compare only the touched rows against an fp64 scatter-add
        acc = np.zeros((len(rows), k))
        pos = np.searchsorted(rows, ir)
        ic = S.ic_h
        np.add.at(acc, pos, data[:, None].astype(np.float64) * B[ic].astype(np.float64))
        assert np.abs(Gs - acc).max() <= 1e-4 * np.abs(acc).max()
        assert float(G.abs().sum()) == pytest.approx(float(np.abs(Gs).sum()), rel=1e-5)   # nothing else was written
        del G, want


def test_single_huge_column_and_single_hot_row(cuda_device, monkeypatch):
    monkeypatch.setenv("BIDMAT_B200_CHUNK", "64")
    rng = np.random.default_rng(3)
    k, m, n = 128, 5000, 9
    jc = np.array([0, 0, 2, 2, 4002, 4003, 4003, 4003, 4010, 4010], dtype=np.int32)
    ir = np.concatenate([[1, 7], np.sort(rng.choice(m, 4000, replace=False)), [7], np.arange(7)]).astype(np.int32)
    data = rng.uniform(0.1, 1, len(ir)).astype(np.float32)
    check_all_ops(k, m, n, jc, ir, data, cuda_device, rng)
    # transpose of it: one hot row shared by every column
    m2, n2 = 11, 3000
    jc2 = np.arange(0, 2 * n2 + 1, 2, dtype=np.int32)
    ir2 = np.stack([np.full(n2, 4), 5 + (np.arange(n2) % 6)], axis=1).flatten().astype(np.int32)
    data2 = rng.uniform(0.1, 1, len(ir2)).astype(np.float32)
    check_all_ops(64, m2, n2, jc2, ir2, data2, cuda_device, rng)


def test_unsorted_and_repeated_rows_inside_columns(cuda_device):
    """GSMat.oneHot / nHot can produce unsorted or repeated rows
    (src/main/scala/BIDMat/GSMat.scala:686-720); results must not depend on
    row order inside a column."""
    rng = np.random.default_rng(11)
    m, n, k = 50, 30, 96
    jc, ir, data = random_csc(m, n, 0.2, rng, sorted_rows=False, dup_rows=True)
    check_all_ops(k, m, n, jc, ir, data, cuda_device, rng)


def test_dds_output_structure_is_bit_identical(cuda_device):
    from bidmat_b200.mat import DDS, GMat, GSMat, SMat
    rng = np.random.default_rng(13)
    m, n, k = 70, 45, 128
    jc, ir, data = random_csc(m, n, 0.2, rng, empty_cols=(2, 44))
    S = SMat(m, n, jc, ir, data).check()
    gs = GSMat.fromSMat(S, cuda_device)
    A = GMat.from_numpy(rng.standard_normal((m, k)).astype(np.float32), cuda_device)
    B = GMat.from_numpy(rng.standard_normal((n, k)).astype(np.float32), cuda_device)
    P = DDS(A, B, gs)
    out = P.toSMat().check()
    assert out.nnz == S.nnz
    assert np.array_equal(out.jc, S.jc) and np.array_equal(out.ir, S.ir)
    assert np.array_equal(P.pic.cpu().numpy(), oracle.uncompress_inds(jc))
    want = oracle.dds(A.to_numpy(), B.to_numpy(), ir, jc)
    _, scale = oracle.dds_f64(A.to_numpy(), B.to_numpy(), ir, jc)
    assert_close_scaled(out.data, want, scale, RTOL_DDS, "DDS via mirror")
    P0 = GSMat.DDS0(A, B, gs)
    assert_close_scaled(P0.pdata.cpu().numpy(), want, scale, RTOL_DDS, "DDS0 via mirror")


def test_results_are_bit_reproducible(cuda_device, monkeypatch):
    monkeypatch.setenv("BIDMAT_B200_CHUNK", "32")
    rng = np.random.default_rng(17)
    m, n, k = 300, 200, 256
    jc, ir, data = random_csc(m, n, 0.3, rng)
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    A = dev(rng.standard_normal((m, k)).astype(np.float32), cuda_device)
    B = dev(rng.standard_normal((n, k)).astype(np.float32), cuda_device)
    runs = []
    for _ in range(3):
        C = abi_dsmult(A, S, torch.zeros((n, k), device=cuda_device))
        G = abi_dsmultT(B, S, torch.zeros((m, k), device=cuda_device))
        P = abi_dds(A, B, S, torch.zeros(S.nnz, device=cuda_device))
        runs.append((C.clone(), G.clone(), P.clone()))
    for r in runs[1:]:
        for a, b in zip(runs[0], r):
            assert torch.equal(a.view(torch.int32), b.view(torch.int32))


def test_empty_inputs_and_bad_arguments(cuda_device):
    from bidmat_b200 import _lib
    L = _lib.lib
    k, m, n = 16, 8, 5
    jc = np.zeros(n + 1, dtype=np.int32)
    S = DeviceCSC(m, n, jc, np.zeros(0, np.int32), np.zeros(0, np.float32), cuda_device)
    A = torch.ones((m, k), device=cuda_device)
    B = torch.ones((n, k), device=cuda_device)
    C = torch.full((n, k), 3.0, device=cuda_device)
    assert L.bidmat_b200_dsmult(k, n, 0, A.data_ptr(), 0, 0, 0, C.data_ptr()) == 0
    assert L.bidmat_b200_dsmultT(k, n, 0, B.data_ptr(), 0, 0, 0, C.data_ptr()) == 0
    assert L.bidmat_b200_dds(k, 0, A.data_ptr(), B.data_ptr(), 0, 0, 0) == 0
    assert L.bidmat_b200_dds0(k, n, A.data_ptr(), B.data_ptr(), 0, S.jc.data_ptr(), 0) == 0
    assert torch.all(C == 3.0)
    assert L.bidmat_b200_dsmult(-1, n, 5, A.data_ptr(), 0, 0, 0, C.data_ptr()) == 1
    assert L.bidmat_b200_dsmult(k, n, 5, 0, 0, 0, 0, 0) == 1
    # the context is still healthy afterwards
    assert float(torch.ones(4, device=cuda_device).sum()) == 4.0


def test_structure_helpers_on_device(cuda_device):
    from bidmat_b200 import _lib
    L = _lib.lib
    rng = np.random.default_rng(23)
    m, n = 64, 200
    jc, ir, data = random_csc(m, n, 0.1, rng, empty_cols=(0, 1, 50, 51, 52, 198, 199))
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    ic = torch.empty(S.nnz, dtype=torch.int32, device=cuda_device)
    assert L.bidmat_b200_expand_jc(n, S.nnz, S.jc.data_ptr(), ic.data_ptr(), 0) == 0
    torch.cuda.synchronize()
    assert np.array_equal(ic.cpu().numpy(), S.ic_h)                    # bit-exact vs uncompressInds
    jc2 = torch.full((n + 1,), -7, dtype=torch.int32, device=cuda_device)
    assert L.bidmat_b200_compress_ic(n, S.nnz, ic.data_ptr(), jc2.data_ptr(), 0) == 0
    torch.cuda.synchronize()
    assert np.array_equal(jc2.cpu().numpy(), jc)                       # bit-exact vs compressInds
    assert L.bidmat_b200_check_structure(m, n, S.nnz, S.ir.data_ptr(), S.ic.data_ptr()) == 0
    assert L.bidmat_b200_check_structure(m - 60, n, S.nnz, S.ir.data_ptr(), S.ic.data_ptr()) == 1
    flipped = torch.flip(S.ic, dims=(0,)).contiguous()
    assert L.bidmat_b200_check_structure(m, n, S.nnz, S.ir.data_ptr(), flipped.data_ptr()) == 1


@pytest.mark.parametrize("m,n,dens", [(10, 20, 0.1), (300, 70, 0.3), (5000, 9000, 0.002), (70000, 40, 0.01)])
def test_device_transpose_is_bit_exact(cuda_device, m, n, dens):
    """GSMatTest "support matrix transpose" (GSMatTest.scala:47-54): aa.t against
    the CPU transpose -- here structure and values must match bit for bit."""
    import scipy.sparse as sp
    from bidmat_b200.mat import GSMat, SMat
    rng = np.random.default_rng(m + n)
    jc, ir, data = random_csc(m, n, dens, rng, empty_cols=(0, n - 1))
    aa = GSMat.fromSMat(SMat(m, n, jc, ir, data).check(), cuda_device)
    bb = aa.t
    assert (bb.nrows, bb.ncols, bb.nnz) == (n, m, len(ir))
    out = bb.toSMat().check()
    ref = sp.csc_matrix((data, ir, jc), shape=(m, n)).T.tocsc()
    ref.sort_indices()
    assert np.array_equal(out.jc, ref.indptr) and np.array_equal(out.ir, ref.indices)
    assert np.array_equal(out.data.view(np.uint32), ref.data.astype(np.float32).view(np.uint32))
    assert np.array_equal(bb.pjc.cpu().numpy(), ref.indptr)
    # transposing twice gives the matrix back
    cc = bb.t.toSMat().check()
    assert np.array_equal(cc.jc, jc) and np.array_equal(cc.ir, ir) and np.array_equal(cc.data, data)


def test_mirror_operators_and_errors(cuda_device):
    from bidmat_b200.mat import GMat, GSMat, Mat, SMat
    rng = np.random.default_rng(29)
    nr, nc, nk = 10, 20, 30                      # GSMatTest.scala:13-16
    jc, ir, data = random_csc(nk, nc, 0.2, rng)
    a = SMat(nk, nc, jc, ir, data).check()
    b = rng.uniform(0, 1, (nk, nr)).astype(np.float32)          # column-major nr x nk
    bb = GMat.from_numpy(b, cuda_device)
    aa = GSMat.fromSMat(a, cuda_device)
    flops0 = Mat.nflops
    cc = bb * aa                                                # nr x nc
    assert Mat.nflops - flops0 == 2 * nr * a.nnz
    d = (a.full().astype(np.float64) @ b.astype(np.float64))    # (nc, nk) @ (nk, nr)
    assert np.abs(cc.to_numpy() - d).max() < 1e-4               # checkSimilar eps
    # *^ : GMat nr x nc  *^  GSMat nk x nc  ->  nr x nk
    e = rng.uniform(0, 1, (nc, nr)).astype(np.float32)
    ee = GMat.from_numpy(e, cuda_device)
    gg = ee.xT(aa)
    dt = a.full().astype(np.float64).T @ e.astype(np.float64)   # (nk, nc) @ (nc, nr)
    assert np.abs(gg.to_numpy() - dt).max() < 1e-4
    # ~ form: accumulate into an existing matrix
    again = bb.madd(aa, cc)
    assert np.abs(again.to_numpy() - 2 * d).max() < 2e-4
    with pytest.raises(RuntimeError, match="GSMult dimensions mismatch"):
        ee * aa
    with pytest.raises(RuntimeError, match="GSMult dimensions mismatch"):
        bb.xT(aa)
    with pytest.raises(RuntimeError, match="dimensions mismatch"):
        GSMat.DDS(ee, bb, aa)        # A would need as many columns as S has rows
    # ^* with a (B @@ S) pair
    A = GMat.from_numpy(rng.standard_normal((nk, 16)).astype(np.float32), cuda_device)
    B = GMat.from_numpy(rng.standard_normal((nc, 16)).astype(np.float32), cuda_device)
    P = A.Tx(B @ aa)
    want = oracle.dds(A.to_numpy(), B.to_numpy(), ir, jc)
    assert np.abs(P.pdata.cpu().numpy() - want).max() < 1e-4
    # colslice gives local, zero-based columns
    sl = aa.colslice(5, 12)
    assert sl.ncols == 7 and int(sl.pjc[0]) == 0 and int(sl.pjc[-1]) == sl.nnz
    if sl.nnz:
        assert int(sl.pic.min()) >= 0 and int(sl.pic.max()) < 7
    part = bb * sl
    assert np.abs(part.to_numpy() - d[5:12]).max() < 1e-4


@pytest.mark.parametrize("k", [32, 64, 128, 256, 512])
def test_generic_kernels_at_the_fast_path_heights(cuda_device, k, monkeypatch):
    """The predicate-free kernels normally take k in {32,...,512}; with the switch
    below the same shapes run through the general kernels, which must agree."""
    monkeypatch.setenv("BIDMAT_B200_GENERIC", "1")
    monkeypatch.setenv("BIDMAT_B200_CHUNK", "64")
    rng = np.random.default_rng(k)
    m, n = 120, 80
    jc, ir, data = random_csc(m, n, 0.25, rng, empty_cols=(5,))
    check_all_ops(k, m, n, jc, ir, data, cuda_device, rng)


@pytest.mark.parametrize("chunk", [0, 32])
@pytest.mark.parametrize("k", [12, 64, 128, 256, 512, 516])
def test_product_and_sampled_product_in_one_pass(cuda_device, k, chunk, monkeypatch):
    """bidmat_b200_dsmult_dds_async: same results as dsmult followed by dds (bit for bit: the
    same arithmetic per output), against the CPU checker, accumulating into non-zero outputs;
    k = 128 / 256 / 512 take the one-pass kernel, the others the two operations in sequence."""
    from gpu_util import L
    if chunk:
        monkeypatch.setenv("BIDMAT_B200_CHUNK", str(chunk))
    rng = np.random.default_rng(900 + k + chunk)
    m, n = 170, 120
    jc, ir, data = random_csc(m, n, 0.25, rng, empty_cols=(0, 7, 119))
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((n, k)).astype(np.float32)
    C0 = rng.standard_normal((n, k)).astype(np.float32)
    P0 = rng.standard_normal(S.nnz).astype(np.float32)
    dA, dB = dev(A, cuda_device), dev(B, cuda_device)
    C, P = dev(C0, cuda_device), dev(P0, cuda_device)
    err = L.bidmat_b200_dsmult_dds_async(k, n, S.nnz, dA.data_ptr(), dB.data_ptr(), S.data.data_ptr(), S.ir.data_ptr(),
                                         S.ic.data_ptr(), C.data_ptr(), P.data_ptr(), None)
    assert err == 0
    torch.cuda.synchronize()
    _, Cabs = oracle.dsmult_f64(A, data, ir, jc)
    _, Pabs = oracle.dds_f64(A, B, ir, jc)
    assert_close_scaled(C.cpu().numpy(), oracle.dsmult(A, data, ir, jc, out=C0.copy()), Cabs + np.abs(C0), RTOL_DSMULT, "one pass: A*S")
    assert_close_scaled(P.cpu().numpy(), oracle.dds(A, B, ir, jc) + P0, Pabs + np.abs(P0), RTOL_DDS, "one pass: DDS")
    C2 = abi_dsmult(dA, S, dev(C0, cuda_device))
    P2 = abi_dds(dA, dB, S, dev(P0, cuda_device))
    assert torch.equal(C.view(torch.int32), C2.view(torch.int32))
    assert_close_scaled(P.cpu().numpy(), P2.cpu().numpy(), Pabs + np.abs(P0), RTOL_DDS, "one pass vs separate DDS")


def test_mirror_product_and_sampled_product_in_one_pass(cuda_device):
    from bidmat_b200.mat import DDS, GMat, GSMat, SMat
    rng = np.random.default_rng(77)
    k, m, n = 256, 90, 60
    jc, ir, data = random_csc(m, n, 0.2, rng)
    S = GSMat.fromSMat(SMat(m, n, jc, ir, data), cuda_device)
    A = GMat.from_numpy(rng.standard_normal((m, k)).astype(np.float32), cuda_device)
    B = GMat.from_numpy(rng.standard_normal((n, k)).astype(np.float32), cuda_device)
    C, P = A.GSMultDDS(B, S)
    assert torch.equal(C.t, (A * S).t)
    assert torch.equal(P.pir, S.pir) and torch.equal(P.pic, S.pic)
    assert torch.allclose(P.pdata, DDS(A, B, S).pdata, rtol=1e-5, atol=1e-5)
