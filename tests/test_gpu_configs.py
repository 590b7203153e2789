"""The five benchmark configurations: reduced sizes against the CPU checker,
config 1 at its full size, and the LDA-shaped configuration at a large size
through size-independent properties (one scalar ties the three operations
together:  <A*S, B> = sum_j data[j]*DDS(A,B,S)[j] = <B*^S, A>)."""
import numpy as np
import pytest
import torch

import oracle
from bidmat_b200 import gen
from util import RTOL_DDS, RTOL_DSMULT, RTOL_DSMULTT, assert_close_scaled, error_summary
from gpu_util import DeviceCSC, abi_dds, abi_dsmult, abi_dsmultT

pytestmark = pytest.mark.gpu


def _report(name, op, rtol, got, want32, want64, scale):
    """Acceptance (rtol * sum|terms| against the fp32 CPU loops), the same bound against the fp64
    oracle, and the figures to report beside them (printed: run pytest with -s to see them)."""
    assert_close_scaled(got, want32, scale, rtol, name + " " + op)
    assert_close_scaled(got, want64, scale, rtol, name + " " + op + " against fp64")
    e = error_summary(got, want32, want64, scale)
    print("PARITY %s | %s | gpu-cpu32 %.2e | gpu-fp64 %.2e | cpu32-fp64 %.2e | max rel (significant, %.0f%%) %.2e"
          % (name, op, e["gpu_vs_cpu32_over_sumabs"], e["gpu_vs_fp64_over_sumabs"], e["cpu32_vs_fp64_over_sumabs"],
             100 * e["significant_fraction"], e["max_rel_err_significant"]))


def run_problem(p, device, check_T=True):
    jc, ir, data = p.jc.cpu().numpy(), p.ir.cpu().numpy(), p.data.cpu().numpy()
    assert oracle.check_csc(p.m, p.n, ir, jc) == 0
    S = DeviceCSC(p.m, p.n, jc, ir, data, device)
    A, B = p.A.to(device), p.B.to(device)
    Ah, Bh = p.A.cpu().numpy(), p.B.cpu().numpy()
    C = abi_dsmult(A, S, torch.zeros((p.n, p.k), device=device)).cpu().numpy()
    C64, Cabs = oracle.dsmult_f64(Ah, data, ir, jc)
    _report(p.name, "A*S", RTOL_DSMULT, C, oracle.dsmult(Ah, data, ir, jc), C64, Cabs)
    P = abi_dds(A, B, S, torch.zeros(S.nnz, device=device)).cpu().numpy()
    P64, Pabs = oracle.dds_f64(Ah, Bh, ir, jc)
    _report(p.name, "DDS", RTOL_DDS, P, oracle.dds(Ah, Bh, ir, jc), P64, Pabs)
    if check_T:
        G = abi_dsmultT(B, S, torch.zeros((p.m, p.k), device=device)).cpu().numpy()
        G64, Gabs = oracle.dsmultT_f64(Bh, data, ir, jc, p.m)
        _report(p.name, "B*^S", RTOL_DSMULTT, G, oracle.dsmultT(Bh, data, ir, jc, p.m), G64, Gabs)


def test_config1_full_size(cuda_device):
    run_problem(gen.config1(1.0, seed=0, device=cuda_device), cuda_device)


def test_config2_and_4_reduced(cuda_device):
    run_problem(gen.config2(0.02, seed=0, device=cuda_device), cuda_device)


@pytest.mark.parametrize("k", [32, 64, 128, 256, 512])
def test_config3_width_sweep_reduced(cuda_device, k):
    run_problem(gen.config3(k, 0.04, seed=0, device=cuda_device), cuda_device, check_T=False)


def test_config5_step_reduced(cuda_device):
    """P = DDS(A,B,S); C = A*S; G = B *^ P (P's values on S's pattern)."""
    p = gen.config5(0.01, seed=0, device=cuda_device)
    run_problem(p, cuda_device)
    jc, ir, data = p.jc.cpu().numpy(), p.ir.cpu().numpy(), p.data.cpu().numpy()
    S = DeviceCSC(p.m, p.n, jc, ir, data, cuda_device)
    A, B = p.A.to(cuda_device), p.B.to(cuda_device)
    P = abi_dds(A, B, S, torch.zeros(S.nnz, device=cuda_device))
    SP = DeviceCSC(p.m, p.n, jc, ir, P.cpu().numpy(), cuda_device)
    G = abi_dsmultT(B, SP, torch.zeros((p.m, p.k), device=cuda_device)).cpu().numpy()
    Bh = p.B.cpu().numpy()
    _, Gabs = oracle.dsmultT_f64(Bh, SP.data_h, ir, jc, p.m)
    assert_close_scaled(G, oracle.dsmultT(Bh, SP.data_h, ir, jc, p.m), Gabs, RTOL_DSMULTT, "config5 G")


def test_lda_shape_large_through_trace_identity(cuda_device):
    """Quarter-size LDA configuration (about 4e7 nonzeros, k = 256): too large
    for the CPU loops in a test, so the three results are tied together by the
    identity above, evaluated in fp64 on the device, plus linearity in the
    sparse values and bit-reproducibility."""
    p = gen.config2(0.25, seed=1, device=cuda_device)
    dev = cuda_device
    n, m, k = p.n, p.m, p.k
    ic = torch.repeat_interleave(torch.arange(n, device=dev, dtype=torch.int32),
                                 (p.jc[1:] - p.jc[:-1]).to(torch.int64))

    class S:
        pass
    S.n, S.nnz, S.ir, S.ic, S.data, S.jc = n, p.nnz, p.ir, ic, p.data, p.jc
    C = abi_dsmult(p.A, S, torch.zeros((n, k), device=dev))
    P = abi_dds(p.A, p.B, S, torch.zeros(p.nnz, device=dev))
    G = abi_dsmultT(p.B, S, torch.zeros((m, k), device=dev))
    t_c = float((C.double() * p.B.double()).sum())
    t_p = float((P.double() * p.data.double()).sum())
    t_g = float((G.double() * p.A.double()).sum())
    scale = float((P.double().abs() * p.data.double()).sum())
    assert abs(t_c - t_p) <= 1e-5 * scale and abs(t_g - t_p) <= 1e-4 * scale, (t_c, t_p, t_g, scale)
    # linearity: doubling the sparse values doubles A*S exactly (power of two)
    S.data = p.data * 2
    C2 = abi_dsmult(p.A, S, torch.zeros((n, k), device=dev))
    assert torch.equal(C2, C * 2)
    # accumulate semantics at scale: a second call adds the same amount again
    C3 = abi_dsmult(p.A, S, C2.clone())
    assert torch.allclose(C3, C2 * 2, rtol=1e-5, atol=0)
    # bit-reproducible transposed product (atomic-free accumulation)
    S.data = p.data
    G2 = abi_dsmultT(p.B, S, torch.zeros((m, k), device=dev))
    assert torch.equal(G.view(torch.int32), G2.view(torch.int32))
    # every row that S never names stays untouched
    touched = torch.zeros(m, dtype=torch.bool, device=dev)
    touched[p.ir.long()] = True
    assert float(G[~touched].abs().sum()) == 0.0
