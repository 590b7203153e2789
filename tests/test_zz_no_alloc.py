"""The allocation-free A*S entry point against the ordinary one.

bidmat_b200_dsmult_noalloc serves hosts that own all device memory themselves
(a caching allocator that has taken the whole GPU) or that cannot tolerate the
device-wide synchronisation of cudaMalloc in a serving loop: its scratch is a
fixed 16 MiB device array inside the library.  The array is shared by all calls
and keeps the previous call's contents, so the test makes two different calls
in a row and compares each with bidmat_b200_dsmult on the same inputs, within
the A*S tolerance used everywhere else (1e-5 of sum|terms|).  The file name
sorts last so that a run stopping at the first failure has already run every
other test.
"""
import numpy as np
import pytest
import torch

import oracle
from util import RTOL_DSMULT, assert_close_scaled, random_csc
from gpu_util import DeviceCSC, abi_dsmult, dev

pytestmark = pytest.mark.gpu


def noalloc_dsmult(A, S, C, stream=0):
    from bidmat_b200 import _lib
    err = _lib.lib.bidmat_b200_dsmult_noalloc(A.shape[1], S.n, S.nnz, A.data_ptr(), S.data.data_ptr(),
                                              S.ir.data_ptr(), S.ic.data_ptr(), C.data_ptr(), stream)
    assert err == 0, _lib.error_string(err)
    torch.cuda.synchronize()
    return C


def _case(k, m, n, density, seed, device, empty=()):
    rng = np.random.default_rng(seed)
    jc, ir, data = random_csc(m, n, density, rng, empty_cols=empty)
    S = DeviceCSC(m, n, jc, ir, data, device)
    A = rng.standard_normal((m, k)).astype(np.float32)
    C0 = rng.standard_normal((n, k)).astype(np.float32)
    return S, A, C0


def test_noalloc_matches_ordinary_entry_point_on_two_calls_in_a_row(cuda_device, monkeypatch):
    monkeypatch.setenv("BIDMAT_B200_CHUNK", "32")       # many chunk-straddling columns -> scratch is really used
    for (k, m, n, density, seed) in ((256, 400, 300, 0.4, 1), (100, 90, 500, 0.3, 2)):
        S, A, C0 = _case(k, m, n, density, seed, cuda_device, empty=(0, 7))
        dA = dev(A, cuda_device)
        want = abi_dsmult(dA, S, dev(C0, cuda_device)).cpu().numpy()
        got = noalloc_dsmult(dA, S, dev(C0, cuda_device)).cpu().numpy()
        _, scale = oracle.dsmult_f64(A, S.data_h, S.ir_h, S.jc_h)
        assert_close_scaled(got, want, scale + np.abs(C0), RTOL_DSMULT, "noalloc vs dsmult k=%d" % k)
        # and against the CPU checker, like every other parity test
        cpu = oracle.dsmult(A, S.data_h, S.ir_h, S.jc_h, out=C0.copy())
        assert_close_scaled(got, cpu, scale + np.abs(C0), RTOL_DSMULT, "noalloc vs CPU k=%d" % k)


def test_noalloc_default_chunking_and_repeatability(cuda_device):
    S, A, C0 = _case(128, 3000, 2000, 0.02, 3, cuda_device)
    dA = dev(A, cuda_device)
    want = abi_dsmult(dA, S, torch.zeros((S.n, 128), device=cuda_device))
    a = noalloc_dsmult(dA, S, torch.zeros((S.n, 128), device=cuda_device))
    b = noalloc_dsmult(dA, S, torch.zeros((S.n, 128), device=cuda_device))
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))          # stale scratch does not leak in
    assert torch.equal(a.view(torch.int32), want.view(torch.int32))       # same chunking -> same bits


def test_noalloc_rejects_problems_beyond_the_fixed_scratch(cuda_device):
    from bidmat_b200 import _lib
    k = 1024
    limit = 16384 * ((4 * 1024 * 1024) // (2 * k))          # 33,554,432 nonzeros at k = 1024
    nnz = limit + 1
    m, n = 8, 4
    ir = torch.zeros(nnz, dtype=torch.int32, device=cuda_device)
    ic = torch.zeros(nnz, dtype=torch.int32, device=cuda_device)
    data = torch.ones(nnz, dtype=torch.float32, device=cuda_device)
    A = torch.ones((m, k), device=cuda_device)
    C = torch.zeros((n, k), device=cuda_device)
    err = _lib.lib.bidmat_b200_dsmult_noalloc(k, n, nnz, A.data_ptr(), data.data_ptr(), ir.data_ptr(),
                                              ic.data_ptr(), C.data_ptr(), 0)
    assert err == 1                                          # cudaErrorInvalidValue, nothing launched
    torch.cuda.synchronize()
    assert float(C.abs().sum()) == 0.0
    # one nonzero fewer is accepted and correct: every term is 1*1 into column 0
    err = _lib.lib.bidmat_b200_dsmult_noalloc(k, n, limit, A.data_ptr(), data.data_ptr(), ir.data_ptr(),
                                              ic.data_ptr(), C.data_ptr(), 0)
    assert err == 0
    torch.cuda.synchronize()
    assert torch.all(C[0] == float(limit)) and float(C[1:].abs().sum()) == 0.0
