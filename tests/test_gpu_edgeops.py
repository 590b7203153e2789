"""Edge operators on GSMat values (sdoprow / sdopcol / spsum) and their mirror
methods, against numpy.  Sums are compared within 1e-5 of sum|terms| and must be
bit-reproducible (no float atomics); element-wise operators must be bit-exact
for the IEEE operations and within 2 ulp for atan2 / pow."""
import numpy as np
import pytest
import torch

from util import random_csc
from gpu_util import DeviceCSC, dev

pytestmark = pytest.mark.gpu


def _np_op(opn, a, b):
    f = [lambda a, b: a + b, lambda a, b: a - b, lambda a, b: a * b, lambda a, b: a / b,
         lambda a, b: (a > b), lambda a, b: (a < b), lambda a, b: (a == b), lambda a, b: (a >= b),
         lambda a, b: (a <= b), lambda a, b: (a != b), np.maximum, np.minimum, np.arctan2, np.power,
         lambda a, b: np.where(a > 0, b, 0)][opn]
    return np.asarray(f(a.astype(np.float32), b.astype(np.float32)), dtype=np.float32)


@pytest.mark.parametrize("opn", list(range(15)))
def test_sdoprow_sdopcol_and_scalar(cuda_device, opn):
    from bidmat_b200 import _lib
    L = _lib.lib
    rng = np.random.default_rng(opn)
    m, n = 90, 70
    jc, ir, data = random_csc(m, n, 0.2, rng)
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    row = rng.uniform(0.2, 2.0, n).astype(np.float32)
    col = rng.uniform(0.2, 2.0, m).astype(np.float32)
    tol = 0 if opn < 12 or opn == 14 else 3e-7
    for (fn, idx_d, idx_h, vec) in ((L.bidmat_b200_sdoprow, S.ic, S.ic_h, row), (L.bidmat_b200_sdopcol, S.ir, S.ir_h, col)):
        A = dev(data.copy(), cuda_device)
        B = dev(vec, cuda_device)
        assert fn(m, n, S.nnz, A.data_ptr(), idx_d.data_ptr(), B.data_ptr(), len(vec), opn) == 0
        want = _np_op(opn, data, vec[idx_h])
        got = A.cpu().numpy()
        assert np.allclose(got, want, rtol=tol, atol=0), (opn, np.abs(got - want).max())
        A = dev(data.copy(), cuda_device)
        assert fn(m, n, S.nnz, A.data_ptr(), idx_d.data_ptr(), B.data_ptr(), 1, opn) == 0
        assert np.allclose(A.cpu().numpy(), _np_op(opn, data, np.full_like(data, vec[0])), rtol=tol, atol=0)
    assert L.bidmat_b200_sdoprow(m, n, S.nnz, S.data.data_ptr(), S.ic.data_ptr(), S.data.data_ptr(), 1, 15) == 1
    assert L.bidmat_b200_sdoprow(m, n, 0, 0, 0, 0, 1, 0) == 0


@pytest.mark.parametrize("m,n,dens", [(50, 40, 0.3), (3000, 2000, 0.01), (7, 50000, 0.3), (600, 700, 0.06), (20000, 37, 0.4)])
def test_spsum_rows_and_columns(cuda_device, m, n, dens, monkeypatch):
    from bidmat_b200 import _lib
    L = _lib.lib
    monkeypatch.setenv("BIDMAT_B200_CHUNK", "64")
    rng = np.random.default_rng(m * 3 + n)
    jc, ir, data = random_csc(m, n, dens, rng, empty_cols=(1,))
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    P = rng.standard_normal(S.nnz).astype(np.float32)
    dP = dev(P, cuda_device)
    for nn, size, idx in ((1, n, S.ic_h), (2, m, S.ir_h)):
        start = rng.standard_normal(size).astype(np.float32)
        outs = []
        for _ in range(2):
            B = dev(start.copy(), cuda_device)
            assert L.bidmat_b200_spsum(m, n, S.nnz, S.ir.data_ptr(), S.ic.data_ptr(), dP.data_ptr(), B.data_ptr(), nn) == 0
            outs.append(B.cpu().numpy())
        want = start.astype(np.float64).copy()
        np.add.at(want, idx, P.astype(np.float64))
        scale = np.abs(start).astype(np.float64)
        np.add.at(scale, idx, np.abs(P).astype(np.float64))
        assert np.all(np.abs(outs[0] - want) <= 1e-5 * scale + 1e-30)
        assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
        # double-precision twin (spsum on doubles, MatKernelD.hpp:51)
        B64 = dev(start.astype(np.float64), cuda_device)
        P64 = dev(P.astype(np.float64), cuda_device)
        assert L.bidmat_b200_spsum_f64(m, n, S.nnz, S.ir.data_ptr(), S.ic.data_ptr(), P64.data_ptr(), B64.data_ptr(), nn) == 0
        assert np.all(np.abs(B64.cpu().numpy() - want) <= 1e-13 * scale + 1e-30)


@pytest.mark.parametrize("skip", [1, 2, 3])
def test_spsum_with_index_and_value_lists_that_start_off_a_16_byte_boundary(cuda_device, skip):
    """The column sums read whole 16-byte vectors only where the lists allow it: lists that start 4, 8 or
    12 bytes into a vector (a view that drops the first nonzeros) take the element-wise loads."""
    from bidmat_b200 import _lib
    L = _lib.lib
    rng = np.random.default_rng(70 + skip)
    m, n = 400, 900
    jc, ir, data = random_csc(m, n, 0.05, rng, empty_cols=(0, 5))
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    P = rng.standard_normal(S.nnz).astype(np.float32)
    dP = dev(P, cuda_device)
    start = rng.standard_normal(n).astype(np.float32)
    B = dev(start.copy(), cuda_device)
    assert L.bidmat_b200_spsum(m, n, S.nnz - skip, S.ir.data_ptr() + 4 * skip, S.ic.data_ptr() + 4 * skip,
                               dP.data_ptr() + 4 * skip, B.data_ptr(), 1) == 0
    want = start.astype(np.float64).copy()
    np.add.at(want, S.ic_h[skip:], P[skip:].astype(np.float64))
    scale = np.abs(start).astype(np.float64)
    np.add.at(scale, S.ic_h[skip:], np.abs(P[skip:]).astype(np.float64))
    assert np.all(np.abs(B.cpu().numpy() - want) <= 1e-5 * scale + 1e-30)


@pytest.mark.parametrize("opn", [0, 2, 3, 10, 13])
def test_double_precision_edge_operators(cuda_device, opn):
    """sdopdrow / sdopdcol (CUMAT.java:137,141): the double overloads."""
    from bidmat_b200 import _lib
    L = _lib.lib
    rng = np.random.default_rng(40 + opn)
    m, n = 60, 45
    jc, ir, data = random_csc(m, n, 0.25, rng)
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    d64 = data.astype(np.float64) + 1e-9
    row, col = rng.uniform(0.2, 2.0, n), rng.uniform(0.2, 2.0, m)
    f = {0: np.add, 2: np.multiply, 3: np.divide, 10: np.maximum, 13: np.power}[opn]
    for fn, idx_d, idx_h, vec in ((L.bidmat_b200_sdoprow_f64, S.ic, S.ic_h, row), (L.bidmat_b200_sdopcol_f64, S.ir, S.ir_h, col)):
        A = dev(d64.copy(), cuda_device)
        B = dev(vec, cuda_device)
        assert fn(m, n, S.nnz, A.data_ptr(), idx_d.data_ptr(), B.data_ptr(), len(vec), opn) == 0
        assert np.allclose(A.cpu().numpy(), f(d64, vec[idx_h]), rtol=(1e-15 if opn != 13 else 1e-14), atol=0)


def test_mirror_sum_and_edge_operators(cuda_device):
    from bidmat_b200.mat import GMat, GSMat, SMat
    rng = np.random.default_rng(8)
    m, n = 40, 30
    jc, ir, data = random_csc(m, n, 0.25, rng)
    a = SMat(m, n, jc, ir, data).check()
    aa = GSMat.fromSMat(a, cuda_device)
    full = a.full().astype(np.float64)                       # (n, m) column-major
    assert np.abs(aa.sum(1).to_numpy()[:, 0] - full.sum(axis=1)).max() < 1e-4     # 1 x n column sums
    assert np.abs(aa.sum(2).to_numpy()[0] - full.sum(axis=0)).max() < 1e-4        # m x 1 row sums
    rowv = GMat.from_numpy(rng.uniform(1, 2, (n, 1)).astype(np.float32), cuda_device)     # 1 x n
    colv = GMat.from_numpy(rng.uniform(1, 2, (1, m)).astype(np.float32), cuda_device)     # m x 1
    ic = np.repeat(np.arange(n), np.diff(jc))
    assert np.array_equal(aa.mul_at(rowv).pdata.cpu().numpy(), data * rowv.to_numpy()[:, 0][ic])
    assert np.array_equal((aa / colv).pdata.cpu().numpy(), data / colv.to_numpy()[0][ir])
    assert np.array_equal(aa.pdata.cpu().numpy(), data)       # operands are not modified
    with pytest.raises(RuntimeError, match="only edge operators"):
        aa + GMat.zeros(m, n, cuda_device)


@pytest.mark.parametrize("nr,nc,kk,offs", [(8, 20, 30, (0, 0, 0, 0, 0, 0)), (12, 17, 23, (3, 5, 7, 11, 2, 4)),
                                           (128, 40, 64, (0, 16, 32, 8, 0, 8)), (130, 33, 50, (1, 2, 3, 4, 5, 6))])
def test_tile_products_against_dense(cuda_device, nr, nc, kk, offs, monkeypatch):
    """GMat.tileMult / tileMultNT with a sparse operand (dsmultTile, dsmultTileT):
    only the nonzeros inside the tile count, everything outside the output tile
    stays untouched, and the product accumulates."""
    from bidmat_b200.mat import GMat, GSMat, SMat
    monkeypatch.setenv("BIDMAT_B200_CHUNK", "32")
    aroff, acoff, broff, bcoff, croff, ccoff = offs
    rng = np.random.default_rng(nr + nc + kk)
    # N: A is (aroff+nr+2) x (acoff+kk+3), S is (broff+kk+4) x (bcoff+nc+5)
    for transpose in (False, True):
        srows, scols = ((nc, kk) if transpose else (kk, nc))
        am, an = aroff + nr + 2, acoff + kk + 3
        sm, sn = broff + srows + 4, bcoff + scols + 5
        cm, cn = croff + nr + 1, ccoff + nc + 2
        jc, ir, data = random_csc(sm, sn, 0.3, rng)
        a_h = rng.standard_normal((an, am)).astype(np.float32)        # column-major am x an
        c0 = rng.standard_normal((cn, cm)).astype(np.float32)
        A = GMat.from_numpy(a_h, cuda_device)
        C = GMat.from_numpy(c0.copy(), cuda_device)
        S = GSMat.fromSMat(SMat(sm, sn, jc, ir, data).check(), cuda_device)
        fn = A.tileMultNT if transpose else A.tileMult
        fn(nr, nc, kk, aroff, acoff, S, broff, bcoff, C, croff, ccoff)
        full = SMat(sm, sn, jc, ir, data).full().astype(np.float64).T          # (sm, sn) row-major dense S
        At = a_h.astype(np.float64).T[aroff:aroff + nr, acoff:acoff + kk]       # nr x kk
        St = full[broff:broff + srows, bcoff:bcoff + scols]
        prod = At @ (St.T if transpose else St)                                 # nr x nc
        want = c0.astype(np.float64).T.copy()                                   # cm x cn
        want[croff:croff + nr, ccoff:ccoff + nc] += prod
        got = C.to_numpy().astype(np.float64).T
        assert np.abs(got - want).max() < 1e-4
        outside = np.ones_like(want, dtype=bool)
        outside[croff:croff + nr, ccoff:ccoff + nc] = False
        assert np.array_equal(got[outside], c0.astype(np.float64).T[outside])
    with pytest.raises(RuntimeError, match="strays outside"):
        A.tileMult(nr, nc, kk, aroff, acoff, S, broff, bcoff + 1000, C, croff, ccoff)
