"""The CUDA path against outputs of the reference's own code:

  * DDS against the stored results of the reference's compiled smcscm / dmcscm
    loop (tests/golden/dds_ref_vectors.npz, made by tests/golden/make_golden.py);
  * every operation against the reference's own CUDA launchers dsmult, dsmultT,
    dds, dds0 and spsum (jni/src/Arith.cu:46-60, 234-248, 381-399, 267-277),
    compiled for sm_100a into oracle/_ref/libarith_ref.so and run on the same
    device buffers.  The reference adds with float atomics, so its own results
    move in the last bits from run to run: values are compared within the
    tolerances of the CPU checker (1e-5 / 1e-4 of sum|terms|), structure exactly.
"""
import os

import numpy as np
import pytest
import torch

import oracle
from util import RTOL_DDS, RTOL_DSMULT, RTOL_DSMULTT, assert_close_scaled, random_csc
from gpu_util import DeviceCSC, L, abi_dds, abi_dds0, abi_dsmult, abi_dsmultT, dev

pytestmark = pytest.mark.gpu

DDS_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "dds_ref_vectors.npz")
needs_ref_gpu = pytest.mark.skipif(not oracle.ref_gpu_available(),
                                   reason="oracle/_ref/libarith_ref.so (reference CUDA build) not present")


@pytest.mark.parametrize("name", ["dds_k1", "dds_k7", "dds_k128", "dds_k130", "dds_k256", "dds_k512"])
def test_dds_against_reference_golden_vectors(cuda_device, name):
    z = np.load(DDS_GOLDEN)
    g = {k.split("/")[1]: z[k] for k in z.files if k.startswith(name + "/")}
    m, n = int(g["m"]), int(g["n"])
    S = DeviceCSC(m, n, g["jc"], g["ir"], np.ones(len(g["ir"]), np.float32), cuda_device)
    _, Pabs = oracle.dds_f64(g["A"], g["B"], g["ir"], g["jc"])
    dA, dB = dev(g["A"], cuda_device), dev(g["B"], cuda_device)
    P = abi_dds(dA, dB, S, torch.zeros(S.nnz, device=cuda_device)).cpu().numpy()
    assert_close_scaled(P, g["P"], Pabs, RTOL_DDS, "golden DDS " + name)
    P0 = abi_dds0(dA, dB, S, torch.full((S.nnz,), 7.0, device=cuda_device)).cpu().numpy()
    assert_close_scaled(P0, g["P"], Pabs, RTOL_DDS, "golden DDS0 " + name)
    # double-precision twin against the dmcscm-derived values
    dA64, dB64 = dA.double(), dB.double()
    P64 = torch.zeros(S.nnz, dtype=torch.float64, device=cuda_device)
    err = L.bidmat_b200_dds_f64(int(g["k"]), S.nnz, dA64.data_ptr(), dB64.data_ptr(), S.ir.data_ptr(),
                                S.ic.data_ptr(), P64.data_ptr())
    assert err == 0
    assert_close_scaled(P64.cpu().numpy(), g["P64"], Pabs, 1e-13, "golden DDS fp64 " + name)


@needs_ref_gpu
@pytest.mark.parametrize("k,m,n,dens", [(32, 200, 150, 0.1), (64, 90, 400, 0.05), (128, 300, 200, 0.1),
                                        (256, 500, 300, 0.08), (512, 120, 100, 0.2), (100, 80, 60, 0.2),
                                        (20, 30, 10, 0.2)])
def test_all_ops_against_the_reference_cuda_kernels(cuda_device, k, m, n, dens):
    rng = np.random.default_rng(1000 + k + m)
    jc, ir, data = random_csc(m, n, dens, rng, empty_cols=(0, n - 1))
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((n, k)).astype(np.float32)
    C0 = rng.standard_normal((n, k)).astype(np.float32)
    G0 = rng.standard_normal((m, k)).astype(np.float32)
    P0 = rng.standard_normal(S.nnz).astype(np.float32)
    dA, dB = dev(A, cuda_device), dev(B, cuda_device)
    ptr = lambda t: t.data_ptr()

    C_ref = dev(C0, cuda_device)
    oracle.ref_gpu_dsmult(k, n, S.nnz, ptr(dA), ptr(S.data), ptr(S.ir), ptr(S.ic), ptr(C_ref))
    C = abi_dsmult(dA, S, dev(C0, cuda_device))
    _, Cabs = oracle.dsmult_f64(A, data, ir, jc)
    assert_close_scaled(C.cpu().numpy(), C_ref.cpu().numpy(), Cabs + np.abs(C0), RTOL_DSMULT, "A*S vs reference kernel")

    G_ref = dev(G0, cuda_device)
    oracle.ref_gpu_dsmultT(k, n, S.nnz, ptr(dB), ptr(S.data), ptr(S.ir), ptr(S.ic), ptr(G_ref))
    G = abi_dsmultT(dB, S, dev(G0, cuda_device))
    _, Gabs = oracle.dsmultT_f64(B, data, ir, jc, m)
    assert_close_scaled(G.cpu().numpy(), G_ref.cpu().numpy(), Gabs + np.abs(G0), RTOL_DSMULTT, "B*^S vs reference kernel")

    if k >= 32:      # the reference's dds uses full-warp shuffles: blocks of min(32, k) x ... threads
        P_ref = dev(P0, cuda_device)
        oracle.ref_gpu_dds(k, S.nnz, ptr(dA), ptr(dB), ptr(S.ir), ptr(S.ic), ptr(P_ref))
        P = abi_dds(dA, dB, S, dev(P0, cuda_device))
        _, Pabs = oracle.dds_f64(A, B, ir, jc)
        assert_close_scaled(P.cpu().numpy(), P_ref.cpu().numpy(), Pabs + np.abs(P0), RTOL_DDS, "DDS vs reference kernel")

    # column and row sums of the values
    for which, length in ((1, n), (2, m)):
        s_ref = torch.zeros(length, device=cuda_device)
        oracle.ref_gpu_spsum(m, n, S.nnz, ptr(S.ir), ptr(S.ic), ptr(S.data), ptr(s_ref), which)
        s = torch.zeros(length, device=cuda_device)
        assert L.bidmat_b200_spsum(m, n, S.nnz, ptr(S.ir), ptr(S.ic), ptr(S.data), ptr(s), which) == 0
        assert torch.allclose(s, s_ref, rtol=1e-5, atol=1e-6)


@needs_ref_gpu
def test_dds0_against_the_reference_kernel_at_its_only_valid_height(cuda_device):
    """The reference's dds0 reads B[tid + k*col] for tid < 1024 whatever k is
    (jni/src/Arith.cu:320-323), so 1024 is the one height at which it is defined."""
    k, m, n = 1024, 40, 130
    rng = np.random.default_rng(5)
    jc, ir, data = random_csc(m, n, 0.2, rng, empty_cols=(7,))
    S = DeviceCSC(m, n, jc, ir, data, cuda_device)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((n, k)).astype(np.float32)
    dA, dB = dev(A, cuda_device), dev(B, cuda_device)
    P_ref = torch.zeros(S.nnz, device=cuda_device)
    oracle.ref_gpu_dds0(k, n, dA.data_ptr(), dB.data_ptr(), S.ir.data_ptr(), S.jc.data_ptr(), P_ref.data_ptr())
    P = abi_dds0(dA, dB, S, torch.zeros(S.nnz, device=cuda_device))
    _, Pabs = oracle.dds_f64(A, B, ir, jc)
    assert_close_scaled(P.cpu().numpy(), P_ref.cpu().numpy(), Pabs, RTOL_DDS, "DDS0 vs reference kernel")
