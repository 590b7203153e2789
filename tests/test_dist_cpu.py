"""Host-side logic of the multi-GPU path on CPU ranks (gloo, world size 2):
columns are split by equal nonzero count, A*S and DDS of the shards concatenate
to the single-rank result bit-exactly, and the B*^S partials summed by one
allreduce match the single-rank result within the B*^S tolerance.  The compute
on each CPU rank is the CPU checker; the CUDA kernels are covered by the GPU
tests."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, scale, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from bidmat_b200 import gen
        from bidmat_b200.step import slice_columns
        from util import RTOL_DSMULTT
        p = gen.config2(scale, seed=3, device="cpu")
        bounds = gen.shard_columns(p.jc, world)
        c0, c1 = bounds[rank], bounds[rank + 1]
        jc, ir, data = (t.numpy() for t in slice_columns(p.jc, p.ir, p.data, c0, c1))
        assert jc[0] == 0 and jc[-1] == len(ir)
        A, B = p.A.numpy(), p.B.numpy()
        C_loc = oracle.dsmult(A, data, ir, jc, nthreads=2)
        P_loc = oracle.dds(A, B[c0:c1], ir, jc, nthreads=2)
        G = torch.from_numpy(oracle.dsmultT(B[c0:c1], data, ir, jc, p.m, nthreads=2))
        dist.all_reduce(G, op=dist.ReduceOp.SUM)
        # gather the (unequal) column blocks
        sizes = [bounds[i + 1] - bounds[i] for i in range(world)]
        nnzs = [int(p.jc[bounds[i + 1]] - p.jc[bounds[i]]) for i in range(world)]
        Cs, Ps = [None] * world, [None] * world
        dist.all_gather_object(Cs, C_loc)
        dist.all_gather_object(Ps, P_loc)
        assert [c.shape[0] for c in Cs] == sizes and [len(x) for x in Ps] == nnzs
        if rank == 0:
            jcf, irf, dataf = p.jc.numpy(), p.ir.numpy(), p.data.numpy()
            C_full = oracle.dsmult(A, dataf, irf, jcf, nthreads=2)
            P_full = oracle.dds(A, B, irf, jcf, nthreads=2)
            G_full = oracle.dsmultT(B, dataf, irf, jcf, p.m, nthreads=2)
            _, Gabs = oracle.dsmultT_f64(B, dataf, irf, jcf, p.m, nthreads=2)
            ok_c = np.array_equal(np.concatenate(Cs), C_full)
            ok_p = np.array_equal(np.concatenate(Ps), P_full)
            ok_g = bool(np.all(np.abs(G.numpy().astype(np.float64) - G_full) <= RTOL_DSMULTT * Gabs + 1e-30))
            balance = max(nnzs) / (sum(nnzs) / world)
            q.put((ok_c, ok_p, ok_g, balance, bounds))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_cpu_ranks_shard_columns_and_allreduce():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 0.004, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    ok_c, ok_p, ok_g, balance, bounds = q.get(timeout=10)
    assert ok_c, "A*S column blocks do not concatenate to the single-rank result"
    assert ok_p, "DDS shards do not concatenate to the single-rank result"
    assert ok_g, "allreduced B*^S partials differ from the single-rank result"
    assert balance < 1.2, (balance, bounds)


def test_shard_columns_properties():
    sys.path.insert(0, ROOT)
    from bidmat_b200 import gen
    jc = torch.tensor([0, 0, 5, 5, 5, 100, 101, 101, 250, 251, 300], dtype=torch.int32)
    for w in (1, 2, 3, 4, 8, 16):
        b = gen.shard_columns(jc, w)
        assert len(b) == w + 1 and b[0] == 0 and b[-1] == 10
        assert all(b[i] <= b[i + 1] for i in range(w))
    empty = torch.zeros(6, dtype=torch.int32)
    assert gen.shard_columns(empty, 4)[-1] == 5
