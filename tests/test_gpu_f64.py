"""Double-precision twins of the four operations (BIDMat's GDMat / GSDMat
path) through the C ABI, against the double-precision CPU loops (pinned to the
reference's dmcscm / dmcsrm).  Tolerance: 1e-13 of sum|terms| for A*S and DDS,
1e-12 for B*^S (same rule as fp32, scaled to the fp64 unit round-off)."""
import numpy as np
import pytest
import scipy.sparse as sp
import torch

import oracle
from util import assert_close_scaled, random_csc
from gpu_util import DeviceCSC, dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("k", [1, 2, 7, 16, 63, 64, 128, 200, 256, 300])
@pytest.mark.parametrize("chunk", [0, 32])
def test_f64_ops(cuda_device, k, chunk, monkeypatch):
    from bidmat_b200 import _lib
    L = _lib.lib
    if chunk:
        monkeypatch.setenv("BIDMAT_B200_CHUNK", str(chunk))
    rng = np.random.default_rng(k * 5 + chunk)
    m, n = 140, 90
    jc, ir, data32 = random_csc(m, n, 0.2, rng, empty_cols=(0, 50))
    data = data32.astype(np.float64) + rng.uniform(0, 1e-9, len(data32))
    S = DeviceCSC(m, n, jc, ir, data32, cuda_device)
    d_data = dev(data, cuda_device)
    A, B = rng.standard_normal((m, k)), rng.standard_normal((n, k))
    C0, G0, P0 = rng.standard_normal((n, k)), rng.standard_normal((m, k)), rng.standard_normal(S.nnz)
    dA, dB = dev(A, cuda_device), dev(B, cuda_device)
    absS = sp.csc_matrix((np.abs(data), ir, jc), shape=(m, n))

    C = dev(C0, cuda_device)
    assert L.bidmat_b200_dsmult_f64(k, n, S.nnz, dA.data_ptr(), d_data.data_ptr(), S.ir.data_ptr(), S.ic.data_ptr(),
                                    C.data_ptr()) == 0
    assert_close_scaled(C.cpu().numpy(), oracle.dsmult_d(A, data, ir, jc, out=C0.copy()),
                        absS.T @ np.abs(A) + np.abs(C0), 1e-13, "f64 A*S")

    G = dev(G0, cuda_device)
    assert L.bidmat_b200_dsmultT_f64(k, n, S.nnz, dB.data_ptr(), d_data.data_ptr(), S.ir.data_ptr(), S.ic.data_ptr(),
                                     G.data_ptr()) == 0
    assert_close_scaled(G.cpu().numpy(), oracle.dsmultT_d(B, data, ir, jc, m, out=G0.copy()),
                        absS @ np.abs(B) + np.abs(G0), 1e-12, "f64 B*^S")

    P = dev(P0, cuda_device)
    assert L.bidmat_b200_dds_f64(k, S.nnz, dA.data_ptr(), dB.data_ptr(), S.ir.data_ptr(), S.ic.data_ptr(),
                                 P.data_ptr()) == 0
    want = oracle.dds_d(A, B, ir, jc)
    scale = np.einsum("ij,ij->i", np.abs(A[ir]), np.abs(B[S.ic_h]))
    assert_close_scaled(P.cpu().numpy(), want + P0, scale + np.abs(P0), 1e-13, "f64 DDS")

    Pz = dev(P0, cuda_device)
    assert L.bidmat_b200_dds0_f64(k, n, dA.data_ptr(), dB.data_ptr(), S.ir.data_ptr(), S.jc.data_ptr(),
                                  Pz.data_ptr()) == 0
    assert_close_scaled(Pz.cpu().numpy(), want, scale, 1e-13, "f64 DDS0")


@pytest.mark.parametrize("k", [64, 256])
def test_f64_transposed_product_with_column_blocks(cuda_device, k, monkeypatch):
    """B*^S in fp64 through the reference-signature entry point with the dense operand cut into
    small column blocks and tiny chunks: the predicate-free kernel on slices of the sorted list."""
    from bidmat_b200 import _lib
    L = _lib.lib
    monkeypatch.setenv("BIDMAT_B200_COLBLOCK_COLS", "32")
    monkeypatch.setenv("BIDMAT_B200_CHUNK", "32")
    rng = np.random.default_rng(300 + k)
    m, n = 70, 150
    jc, ir, data32 = random_csc(m, n, 0.3, rng, empty_cols=(0, 149))
    data = data32.astype(np.float64) + rng.uniform(0, 1e-9, len(data32))
    S = DeviceCSC(m, n, jc, ir, data32, cuda_device)
    B = rng.standard_normal((n, k))
    G0 = rng.standard_normal((m, k))
    G, dB, dd = dev(G0, cuda_device), dev(B, cuda_device), dev(data, cuda_device)
    assert L.bidmat_b200_dsmultT_f64(k, n, S.nnz, dB.data_ptr(), dd.data_ptr(), S.ir.data_ptr(), S.ic.data_ptr(),
                                     G.data_ptr()) == 0
    absS = sp.csc_matrix((np.abs(data), ir, jc), shape=(m, n))
    assert_close_scaled(G.cpu().numpy(), oracle.dsmultT_d(B, data, ir, jc, m, out=G0.copy()),
                        absS @ np.abs(B) + np.abs(G0), 1e-12, "f64 B*^S in column blocks")


def test_f64_results_are_bit_reproducible_and_noop_on_empty(cuda_device, monkeypatch):
    from bidmat_b200 import _lib
    L = _lib.lib
    monkeypatch.setenv("BIDMAT_B200_CHUNK", "32")
    rng = np.random.default_rng(1)
    m, n, k = 200, 150, 96
    jc, ir, data32 = random_csc(m, n, 0.3, rng)
    S = DeviceCSC(m, n, jc, ir, data32, cuda_device)
    d_data = dev(data32.astype(np.float64), cuda_device)
    B = dev(rng.standard_normal((n, k)), cuda_device)
    outs = []
    for _ in range(2):
        G = torch.zeros((m, k), dtype=torch.float64, device=cuda_device)
        assert L.bidmat_b200_dsmultT_f64(k, n, S.nnz, B.data_ptr(), d_data.data_ptr(), S.ir.data_ptr(),
                                         S.ic.data_ptr(), G.data_ptr()) == 0
        outs.append(G)
    assert torch.equal(outs[0].view(torch.int64), outs[1].view(torch.int64))
    assert L.bidmat_b200_dsmult_f64(k, n, 0, 0, 0, 0, 0, 0) == 0
    assert L.bidmat_b200_dds_f64(k, 0, 0, 0, 0, 0, 0) == 0
