"""Two GPUs (skipped on a single-GPU machine): the library's peer-memory sum of
the B*^S partials gives the same bits as NCCL's allreduce for two ranks, every
rank ends with identical G, and the sharded step matches the CPU checker."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from datetime import timedelta
    # a lone rank gives up instead of waiting inside a collective for a peer that died
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=timedelta(seconds=120))
    try:
        from bidmat_b200 import gen, step as pstep
        p = gen.config2(0.03, seed=5, device=dev)
        shard, _ = pstep.make_shard(p, rank, world)
        B_local = p.B[shard.col0:shard.col1].contiguous()
        stream = torch.cuda.Stream(device=dev)
        outs = {}
        kinds = {}
        with torch.cuda.stream(stream):
            # NCCL; the library's sum through the switch (where the buffers have a multicast
            # mapping); the library's sum over peer loads and stores of the touched rows
            for mode, peer, mc, parts in (("nccl", False, "0", "0"), ("switch", True, "1", "0"), ("rows", True, "0", "0"),
                                          ("rows_in_parts", True, "0", "4"), ("switch_in_parts", True, "1", "3")):
                os.environ["BIDMAT_B200_PEER_MC"] = mc
                os.environ["BIDMAT_B200_PIPE_PARTS"] = parts
                st = pstep.PathStep(p.k, shard, p.A, B_local, stream, dist.group.WORLD, peer_reduce=peer)
                in_parts = " in %d parts" % (len(st.parts) - 1) if st.parts else ""
                kinds[mode] = ("switch" + in_parts) if st.mc else (("rows" + in_parts) if st.touched is not None
                                                                   else "nccl" if st.peer is None else "dense")
                for _ in range(3):        # several steps: the buffers are reused from step to step
                    st.run()
                torch.cuda.synchronize()
                dist.barrier()
                outs[mode] = st.G.clone()
                st.close()
        # two ranks: a + b in every implementation
        same_bits = all(torch.equal(outs["nccl"], outs[x]) for x in ("switch", "rows", "rows_in_parts", "switch_in_parts"))
        same_across_ranks = True
        for mode in ("switch", "rows", "rows_in_parts", "switch_in_parts"):
            other = outs[mode].clone()
            dist.broadcast(other, src=0)
            same_across_ranks = same_across_ranks and torch.equal(other.view(torch.int32), outs[mode].view(torch.int32))
        outs[True] = outs["rows"]
        if rank == 0:
            print("allreduce kinds exercised:", kinds, flush=True)
        if rank == 0:
            import oracle
            from util import RTOL_DSMULTT
            jc, ir, data = p.jc.cpu().numpy(), p.ir.cpu().numpy(), p.data.cpu().numpy()
            Bh = p.B.cpu().numpy()
            want = oracle.dsmultT(Bh, data, ir, jc, p.m)
            _, scale = oracle.dsmultT_f64(Bh, data, ir, jc, p.m)
            ok = bool(np.all(np.abs(outs[True].cpu().numpy().astype(np.float64) - want) <= RTOL_DSMULTT * scale + 1e-30))
            q.put((rank, same_bits, same_across_ranks, ok))
        else:
            q.put((rank, same_bits, same_across_ranks, True))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.timeout(600)
def test_peer_memory_sum_matches_nccl_on_two_gpus():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        results = {}
        for _ in procs:
            r = q.get(timeout=500)            # every rank reports: a missing report is a failure
            results[r[0]] = r[1:]
        for p in procs:
            p.join(60)
    finally:
        for p in procs:                       # never leave a child spinning on the device
            if p.is_alive():
                p.kill()
                p.join()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert sorted(results) == [0, 1]
    for rank, (same_bits, same_across_ranks, ok) in results.items():
        assert same_bits, "rank %d: peer-memory sum and NCCL allreduce differ for two ranks" % rank
        assert same_across_ranks, "rank %d: ranks ended with different G" % rank
        assert ok, "sharded B*^S differs from the CPU checker"
