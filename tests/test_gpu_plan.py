"""The prepared transposed product (bidmat_b200_dsmultT_plan_create / _planned) through
the C ABI: parity with the CPU checker, agreement with the unprepared entry point,
overwrite mode, bit-reproducibility, exact structure verification and misuse."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from bidmat_b200 import _lib
from util import RTOL_DSMULTT, assert_close_scaled, random_csc
from gpu_util import DeviceCSC, L, abi_dsmultT, dev

pytestmark = pytest.mark.gpu

OVERWRITE = 1
INFO = ("nnz", "ncols", "m", "k", "elem_bytes", "blocks", "chunks", "split_runs", "slots", "cleared_rows",
        "touched_rows", "bytes", "row_runs")


class Plan:
    def __init__(self, k, S, elem=4):
        self.h = ctypes.c_void_p(0)
        err = L.bidmat_b200_dsmultT_plan_create(k, S.n, S.nnz, S.m, S.ir.data_ptr(), S.ic.data_ptr(), elem, None,
                                                ctypes.byref(self.h))
        assert err == 0, _lib.error_string(err)

    def info(self):
        out = (ctypes.c_longlong * len(INFO))()
        assert L.bidmat_b200_plan_info(self.h, out, len(INFO)) == 0
        return dict(zip(INFO, [int(v) for v in out]))

    def run(self, B, S, G, flags=0, data=None):
        k = B.shape[1]
        fn = L.bidmat_b200_dsmultT_planned if B.dtype == torch.float32 else L.bidmat_b200_dsmultT_planned_f64
        err = fn(self.h, k, S.n, S.nnz, B.data_ptr(), (S.data if data is None else data).data_ptr(), G.data_ptr(),
                 flags, None)
        assert err == 0, _lib.error_string(err)
        torch.cuda.synchronize()
        return G

    def close(self):
        assert L.bidmat_b200_plan_destroy(self.h) == 0


def check_planned(k, m, n, jc, ir, data, device, rng):
    S = DeviceCSC(m, n, jc, ir, data, device)
    B = rng.standard_normal((n, k)).astype(np.float32)
    G0 = rng.standard_normal((m, k)).astype(np.float32)
    dB = dev(B, device)
    plan = Plan(k, S)
    info = plan.info()
    assert info["nnz"] == S.nnz and info["m"] == m and info["k"] == k
    assert info["touched_rows"] == len(np.unique(ir))
    # accumulate
    G = plan.run(dB, S, dev(G0, device)).cpu().numpy()
    Gw = oracle.dsmultT(B, data, ir, jc, m, out=G0.copy())
    _, Gabs = oracle.dsmultT_f64(B, data, ir, jc, m)
    assert_close_scaled(G, Gw, Gabs + np.abs(G0), RTOL_DSMULTT, "planned B*^S k=%d" % k)
    # overwrite: touched rows hold the product, the others keep what they had
    Go = plan.run(dB, S, dev(G0, device), OVERWRITE).cpu().numpy()
    touched = np.zeros(m, bool)
    touched[ir] = True
    Gz = oracle.dsmultT(B, data, ir, jc, m)
    assert_close_scaled(Go[touched], Gz[touched], Gabs[touched], RTOL_DSMULTT, "planned overwrite k=%d" % k)
    assert np.array_equal(Go[~touched], G0[~touched])
    # touched-row bitmap
    bm = torch.zeros((m + 31) // 32, dtype=torch.int32, device=device)
    assert L.bidmat_b200_plan_touched_rows(plan.h, bm.data_ptr(), None) == 0
    torch.cuda.synchronize()
    bits = np.unpackbits(bm.cpu().numpy().view(np.uint8), bitorder="little")[:m].astype(bool)
    assert np.array_equal(bits, touched)
    # new values on the same structure, same plan; bit-identical on repetition
    data2 = (data * 3 + 1).astype(np.float32)
    d2 = dev(data2, device)
    G2 = plan.run(dB, S, torch.zeros((m, k), device=device), 0, d2)
    G2b = plan.run(dB, S, torch.zeros((m, k), device=device), 0, d2)
    assert torch.equal(G2.view(torch.int32), G2b.view(torch.int32))
    _, G2abs = oracle.dsmultT_f64(B, data2, ir, jc, m)
    assert_close_scaled(G2.cpu().numpy(), oracle.dsmultT(B, data2, ir, jc, m), G2abs, RTOL_DSMULTT, "planned, new values")
    plan.close()
    return info


@pytest.mark.parametrize("k", [1, 7, 32, 64, 100, 128, 256, 260, 512, 640])
def test_planned_product_over_dense_heights(cuda_device, k):
    rng = np.random.default_rng(300 + k)
    m, n = 140, 90
    jc, ir, data = random_csc(m, n, 0.15, rng, empty_cols=(0, 5, 89))
    check_planned(k, m, n, jc, ir, data, cuda_device, rng)


@pytest.mark.parametrize("chunk", [8, 32, 96])
@pytest.mark.parametrize("cols_per_block", [0, 4, 16])
@pytest.mark.parametrize("k", [12, 128, 256])
def test_planned_product_with_split_runs_and_column_blocks(cuda_device, k, chunk, cols_per_block, monkeypatch):
    """Tiny chunks split the long rows over many chunks (pieces in slots, one fix-up at the
    end); tiny forced column blocks give every row several runs, a first block to store into
    in overwrite mode, and rows whose first run is split (cleared instead)."""
    monkeypatch.setenv("BIDMAT_B200_CHUNK", str(chunk))
    if cols_per_block:
        monkeypatch.setenv("BIDMAT_B200_COLBLOCK_COLS", str(cols_per_block))
    rng = np.random.default_rng(k + chunk + cols_per_block)
    m, n = 50, 70
    jc, ir, data = random_csc(m, n, 0.5, rng, empty_cols=(3,))
    info = check_planned(k, m, n, jc, ir, data, cuda_device, rng)
    assert info["slots"] >= 2 * info["split_runs"]
    if cols_per_block:
        assert info["blocks"] > 1
    elif chunk <= 32:
        assert info["split_runs"] > 0 and info["cleared_rows"] > 0


@pytest.mark.parametrize("k", [64, 256])
def test_rows_split_in_every_column_block(cuda_device, k, monkeypatch):
    """A few long rows over many columns with small column blocks and chunks: every row is
    split in every block, so one row has many split runs whose totals must be added by one
    worker (a per-run update of the output would race).  Repeated to expose a race."""
    monkeypatch.setenv("BIDMAT_B200_CHUNK", "8")
    monkeypatch.setenv("BIDMAT_B200_COLBLOCK_COLS", "64")
    rng = np.random.default_rng(k)
    m, n = 6, 1500
    jc, ir, data = random_csc(m, n, 0.85, rng)
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    B = rng.standard_normal((n, k)).astype(np.float32)
    dB = dev(B, cuda_device)
    plan = Plan(k, S)
    info = plan.info()
    assert info["blocks"] >= 20 and info["split_runs"] >= 5 * info["blocks"]
    want = oracle.dsmultT(B, data, ir, jc, m)
    _, Gabs = oracle.dsmultT_f64(B, data, ir, jc, m)
    first = None
    for rep in range(20):
        for flags in (0, OVERWRITE):
            G = plan.run(dB, S, torch.zeros((m, k), device=cuda_device), flags)
            assert_close_scaled(G.cpu().numpy(), want, Gabs, RTOL_DSMULTT, "split in every block, rep %d" % rep)
            if first is None:
                first = G.clone()
            assert torch.equal(first.view(torch.int32), G.view(torch.int32))
    plan.close()


def test_planned_product_on_skewed_rows(cuda_device):
    """Zipf rows (a few very long rows, many rows with one nonzero): the shape the chunk
    layout is made for.  Also checks the unprepared entry point against the same result."""
    from bidmat_b200 import gen
    p = gen.config2(0.02, seed=3, device=cuda_device)
    jc, ir, data = p.jc.cpu().numpy(), p.ir.cpu().numpy(), p.data.cpu().numpy()
    S = DeviceCSC(p.m, p.n, jc, ir, data, cuda_device)
    plan = Plan(p.k, S)
    G = plan.run(p.B, S, torch.zeros((p.m, p.k), device=cuda_device))
    Bh = p.B.cpu().numpy()
    _, Gabs = oracle.dsmultT_f64(Bh, data, ir, jc, p.m)
    assert_close_scaled(G.cpu().numpy(), oracle.dsmultT(Bh, data, ir, jc, p.m), Gabs, RTOL_DSMULTT, "planned, Zipf rows")
    Gd = abi_dsmultT(p.B, S, torch.zeros((p.m, p.k), device=cuda_device))
    assert_close_scaled(G.cpu().numpy(), Gd.cpu().numpy(), Gabs, RTOL_DSMULTT, "planned vs unprepared")
    plan.close()


def test_planned_product_double_precision(cuda_device):
    rng = np.random.default_rng(11)
    k, m, n = 96, 80, 60
    jc, ir, data = random_csc(m, n, 0.2, rng)
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    B = rng.standard_normal((n, k))
    d64 = data.astype(np.float64)
    plan = Plan(k, S, elem=8)
    G = plan.run(dev(B, cuda_device), S, torch.zeros((m, k), dtype=torch.float64, device=cuda_device), 0,
                 dev(d64, cuda_device))
    want = oracle.dsmultT_d(B, d64, ir, jc, m)
    assert np.allclose(G.cpu().numpy(), want, rtol=1e-12, atol=1e-12)
    plan.close()


@pytest.mark.parametrize("k", [16, 64, 128, 256])
@pytest.mark.parametrize("chunk,colblock", [(0, 0), (32, 16)])
def test_planned_product_double_precision_at_the_predicate_free_heights(cuda_device, k, chunk, colblock, monkeypatch):
    """k = 2*lanes*vectors in fp64 takes the predicate-free plan kernel (values permuted by a pass of
    their own); tiny chunks and column blocks force split runs, slots and both fix-up levels."""
    if chunk:
        monkeypatch.setenv("BIDMAT_B200_CHUNK", str(chunk))
    if colblock:
        monkeypatch.setenv("BIDMAT_B200_COLBLOCK_COLS", str(colblock))
    rng = np.random.default_rng(100 + k + chunk)
    m, n = 90, 130
    jc, ir, data = random_csc(m, n, 0.35, rng, empty_cols=(3, 77))
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    B = rng.standard_normal((n, k))
    G0 = rng.standard_normal((m, k))
    d64 = data.astype(np.float64) + rng.uniform(0, 1e-9, len(data))
    dd = dev(d64, cuda_device)
    plan = Plan(k, S, elem=8)
    absS = np.zeros((m, n))
    np.add.at(absS, (ir, S.ic_h), np.abs(d64))
    scale = absS @ np.abs(B)
    dB = dev(B, cuda_device)
    G = plan.run(dB, S, dev(G0, cuda_device), 0, dd).cpu().numpy()
    want = oracle.dsmultT_d(B, d64, ir, jc, m, out=G0.copy())
    assert_close_scaled(G, want, scale + np.abs(G0), 1e-12, "planned f64 B*^S k=%d" % k)
    # overwrite mode on a dirty buffer: rows the matrix touches equal the product, the others keep their contents
    Gd = plan.run(dB, S, dev(G0, cuda_device), OVERWRITE, dd).cpu().numpy()
    want0 = oracle.dsmultT_d(B, d64, ir, jc, m)
    touched = np.zeros(m, dtype=bool)
    touched[ir] = True
    assert_close_scaled(Gd[touched], want0[touched], scale[touched], 1e-12, "planned f64 overwrite k=%d" % k)
    assert np.array_equal(Gd[~touched], G0[~touched])
    # same bits on a second run
    G2 = plan.run(dB, S, dev(G0, cuda_device), 0, dd).cpu().numpy()
    assert np.array_equal(G.view(np.int64), G2.view(np.int64))
    plan.close()


def test_plan_verification_and_misuse(cuda_device):
    rng = np.random.default_rng(4)
    k, m, n = 64, 40, 30
    jc, ir, data = random_csc(m, n, 0.3, rng)
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    plan = Plan(k, S)
    assert L.bidmat_b200_plan_verify(plan.h, S.n, S.nnz, S.ir.data_ptr(), S.ic.data_ptr(), None) == 0
    # one row index changed: same sizes, different structure
    ir2 = S.ir.clone()
    ir2[S.nnz // 2] = (int(ir2[S.nnz // 2]) + 1) % m
    assert L.bidmat_b200_plan_verify(plan.h, S.n, S.nnz, ir2.data_ptr(), S.ic.data_ptr(), None) == 1
    B = torch.zeros((n, k), device=cuda_device)
    G = torch.zeros((m, k), device=cuda_device)
    # sizes that are not the plan's: refused with cudaErrorInvalidValue, nothing launched
    n0 = L.bidmat_b200_launch_count()
    assert L.bidmat_b200_dsmultT_planned(plan.h, k, S.n, S.nnz - 1, B.data_ptr(), S.data.data_ptr(), G.data_ptr(), 0, None) == 1
    assert L.bidmat_b200_dsmultT_planned(plan.h, k, S.n + 1, S.nnz, B.data_ptr(), S.data.data_ptr(), G.data_ptr(), 0, None) == 1
    assert L.bidmat_b200_dsmultT_planned(plan.h, k * 2, S.n, S.nnz, B.data_ptr(), S.data.data_ptr(), G.data_ptr(), 0, None) == 1
    assert L.bidmat_b200_dsmultT_planned_f64(plan.h, k, S.n, S.nnz, B.data_ptr(), S.data.data_ptr(), G.data_ptr(), 0, None) == 1
    assert L.bidmat_b200_dsmultT_planned(plan.h, k, S.n, S.nnz, B.data_ptr(), S.data.data_ptr(), G.data_ptr(), 8, None) == 1
    assert L.bidmat_b200_launch_count() == n0
    h = ctypes.c_void_p(0)
    assert L.bidmat_b200_dsmultT_plan_create(k, S.n, 0, m, S.ir.data_ptr(), S.ic.data_ptr(), 4, None, ctypes.byref(h)) == 1
    assert L.bidmat_b200_dsmultT_plan_create(k, S.n, S.nnz, m, S.ir.data_ptr(), S.ic.data_ptr(), 2, None, ctypes.byref(h)) == 1
    plan.close()
    assert L.bidmat_b200_plan_destroy(None) == 0


def test_mirror_keeps_the_plan_on_the_matrix(cuda_device):
    """GSMat.prepareT: later `B *^ S` and `B *^ DDS(A,B,S)` go through the plan."""
    from bidmat_b200.mat import DDS, GMat, GSMat, Mat, SMat
    rng = np.random.default_rng(21)
    k, m, n = 128, 70, 50
    jc, ir, data = random_csc(m, n, 0.2, rng)
    S = GSMat.fromSMat(SMat(m, n, jc, ir, data), cuda_device).prepareT(k)
    A = GMat.from_numpy(rng.standard_normal((m, k)).astype(np.float32), cuda_device)
    B = GMat.from_numpy(rng.standard_normal((n, k)).astype(np.float32), cuda_device)
    Mat.debugStructure = True
    try:
        G = B.xT(S).to_numpy()
        P = DDS(A, B, S)
        assert P._plans is S._plans
        G2 = B.xT(P).to_numpy()
    finally:
        Mat.debugStructure = False
    Bh = B.to_numpy()
    _, Gabs = oracle.dsmultT_f64(Bh, data, ir, jc, m)
    assert_close_scaled(G, oracle.dsmultT(Bh, data, ir, jc, m), Gabs, RTOL_DSMULTT, "mirror planned")
    Ph = P.pdata.cpu().numpy()
    _, G2abs = oracle.dsmultT_f64(Bh, Ph, ir, jc, m)
    assert_close_scaled(G2, oracle.dsmultT(Bh, Ph, ir, jc, m), G2abs, RTOL_DSMULTT, "mirror planned on DDS result")
    S.dropPlans()


def test_workspace_limit_refuses_on_the_host_and_leaves_the_library_usable(cuda_device):
    rng = np.random.default_rng(8)
    k, m, n = 64, 300, 200
    jc, ir, data = random_csc(m, n, 0.2, rng)
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    B = dev(rng.standard_normal((n, k)).astype(np.float32), cuda_device)
    G = torch.zeros((m, k), device=cuda_device)
    assert L.bidmat_b200_set_workspace_limit(1024) == 0
    try:
        n0 = L.bidmat_b200_launch_count()
        err = L.bidmat_b200_dsmultT(k, S.n, S.nnz, B.data_ptr(), S.data.data_ptr(), S.ir.data_ptr(), S.ic.data_ptr(),
                                    G.data_ptr())
        assert err == 2, err                      # cudaErrorMemoryAllocation
        assert L.bidmat_b200_launch_count() == n0 and float(G.abs().sum()) == 0.0
    finally:
        assert L.bidmat_b200_set_workspace_limit(0) == 0
    Gd = abi_dsmultT(B, S, G).cpu().numpy()         # the same call goes through once the limit is lifted
    _, Gabs = oracle.dsmultT_f64(B.cpu().numpy(), data, ir, jc, m)
    assert_close_scaled(Gd, oracle.dsmultT(B.cpu().numpy(), data, ir, jc, m), Gabs, RTOL_DSMULTT, "after limit")
    assert L.bidmat_b200_workspace_bytes() > 0
    assert L.bidmat_b200_release_workspace() == 0


def _auto_info():
    out = (ctypes.c_longlong * 6)()
    assert L.bidmat_b200_auto_plan_info(out, 6) == 0
    return dict(zip(("enabled", "built", "planned_calls", "plain_calls", "kept", "bytes"), [int(v) for v in out]))


def test_plans_kept_by_the_library_behind_the_reference_signature(cuda_device):
    """bidmat_b200_set_auto_plan: the synchronous natives recognise a structure by its fingerprint,
    build a plan at the second sighting and use it from then on; other structures, other heights
    and structures seen once take the ordinary path; results as the ordinary path's."""
    rng = np.random.default_rng(21)
    k, m, n = 128, 300, 260
    jc, ir, data = random_csc(m, n, 0.1, rng, empty_cols=(7,))
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    B = rng.standard_normal((n, k)).astype(np.float32)
    G0 = rng.standard_normal((m, k)).astype(np.float32)
    dB = dev(B, cuda_device)
    want = oracle.dsmultT(B, data, ir, jc, m, out=G0.copy())
    _, scale = oracle.dsmultT_f64(B, data, ir, jc, m)

    def call(Sx, values=None, kk=k, dBx=None):
        G = dev(G0[:, :kk].copy() if kk != k else G0, cuda_device)
        vals = Sx.data if values is None else values
        assert L.bidmat_b200_dsmultT(kk, Sx.n, Sx.nnz, (dB if dBx is None else dBx).data_ptr(), vals.data_ptr(),
                                     Sx.ir.data_ptr(), Sx.ic.data_ptr(), G.data_ptr()) == 0
        return G.cpu().numpy()

    plain = call(S)                                    # switched off: the ordinary path
    assert _auto_info()["enabled"] == 0
    assert L.bidmat_b200_set_auto_plan(1) == 0
    try:
        base = _auto_info()
        outs = [call(S) for _ in range(4)]
        info = _auto_info()
        assert info["built"] - base["built"] == 1 and info["kept"] == 1 and info["bytes"] > 0
        assert info["plain_calls"] - base["plain_calls"] == 1 and info["planned_calls"] - base["planned_calls"] == 3
        for G in outs:
            assert_close_scaled(G, want, scale + np.abs(G0), RTOL_DSMULTT, "kept plan")
        assert np.array_equal(outs[0].view(np.uint32), plain.view(np.uint32))          # first sighting: ordinary path
        assert np.array_equal(outs[1].view(np.uint32), outs[3].view(np.uint32))          # planned calls repeat bit for bit
        # other values on the same structure (a DDS result): same plan
        data2 = rng.standard_normal(S.nnz).astype(np.float32)
        G2 = call(S, dev(data2, cuda_device))
        _, scale2 = oracle.dsmultT_f64(B, data2, ir, jc, m)
        assert_close_scaled(G2, oracle.dsmultT(B, data2, ir, jc, m, out=G0.copy()), scale2 + np.abs(G0), RTOL_DSMULTT,
                            "kept plan, other values")
        assert _auto_info()["planned_calls"] - base["planned_calls"] == 4
        # a different structure of the same sizes: rows of two nonzeros of one column exchanged with unused rows
        ir3 = ir.copy()
        c = int(np.argmax(np.diff(jc)))
        free = np.setdiff1d(np.arange(m), ir[jc[c]:jc[c + 1]])[:2]
        ir3[jc[c]:jc[c] + 2] = free
        S3 = DeviceCSC(m, n, jc, ir3, data, cuda_device)
        before = _auto_info()
        G3 = call(S3)
        after = _auto_info()
        assert after["plain_calls"] - before["plain_calls"] == 1 and after["built"] == before["built"]
        _, scale3 = oracle.dsmultT_f64(B, data, ir3, jc, m)
        assert_close_scaled(G3, oracle.dsmultT(B, data, ir3, jc, m, out=G0.copy()), scale3 + np.abs(G0), RTOL_DSMULTT,
                            "other structure")
        # structures that come by once never cost a plan and do not push the kept one out
        for i in range(10):
            jcx, irx, datax = random_csc(m, n, 0.1, np.random.default_rng(1000 + i))
            Sx = DeviceCSC(m, n, jcx, irx, datax, cuda_device)
            Gx = call(Sx)
            _, sx = oracle.dsmultT_f64(B, datax, irx, jcx, m)
            assert_close_scaled(Gx, oracle.dsmultT(B, datax, irx, jcx, m, out=G0.copy()), sx + np.abs(G0), RTOL_DSMULTT,
                                "passing structure %d" % i)
        assert _auto_info()["built"] == after["built"]
        before = _auto_info()
        assert np.array_equal(call(S).view(np.uint32), outs[1].view(np.uint32))
        assert _auto_info()["planned_calls"] - before["planned_calls"] == 1
        # the double-precision native keeps plans of its own
        B64, d64, G064 = B.astype(np.float64), data.astype(np.float64), G0.astype(np.float64)
        dB64, dd64 = dev(B64, cuda_device), dev(d64, cuda_device)
        for i in range(3):
            G = dev(G064, cuda_device)
            assert L.bidmat_b200_dsmultT_f64(k, n, S.nnz, dB64.data_ptr(), dd64.data_ptr(), S.ir.data_ptr(),
                                             S.ic.data_ptr(), G.data_ptr()) == 0
            assert_close_scaled(G.cpu().numpy(), oracle.dsmultT_d(B64, d64, ir, jc, m, out=G064.copy()),
                                scale + np.abs(G064), 1e-12, "kept plan, fp64, call %d" % i)
        assert _auto_info()["kept"] == 2
    finally:
        assert L.bidmat_b200_set_auto_plan(0) == 0
    info = _auto_info()
    assert info["enabled"] == 0 and info["kept"] == 0 and info["bytes"] == 0
