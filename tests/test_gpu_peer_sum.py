"""The library's sum of the B*^S partials over ranks (csrc/peer_reduce.cu, the replacement of
GFunctions.ncclAllReduce, GFunctions.scala:175-203) on ONE GPU: the buffers of all "ranks" live
on the same device and every rank's call is made in turn.  The kernels never wait for another
rank (rank r reduces slice r of all buffers and stores the total into all of them), so calling
the ranks one after the other computes exactly what W GPUs compute at once.  The two-GPU test
of the same kernels over NVLink is tests/test_gpu_multi.py."""
import ctypes

import numpy as np
import pytest
import torch

from gpu_util import L

pytestmark = pytest.mark.gpu


def _addresses(bufs):
    return (ctypes.c_ulonglong * len(bufs))(*[b.data_ptr() for b in bufs])


def _sum_in_rank_order(parts):
    acc = parts[0].copy()
    for p in parts[1:]:
        acc += p                      # float32, rank 0 first: the kernel's order
    return acc


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("k,m", [(4, 37), (64, 1001), (256, 300)])
def test_peer_sum_over_whole_buffers(cuda_device, world, k, m):
    rng = np.random.default_rng(world * 100 + k)
    host = [rng.standard_normal((m, k)).astype(np.float32) for _ in range(world)]
    bufs = [torch.from_numpy(h).to(cuda_device) for h in host]
    addrs = _addresses(bufs)
    for r in range(world):
        assert L.bidmat_b200_peer_allreduce_sum(world, r, addrs, m * k, 5, None) == 0
    torch.cuda.synchronize()
    want = _sum_in_rank_order(host)
    for r in range(world):
        assert np.array_equal(bufs[r].cpu().numpy().view(np.uint32), want.view(np.uint32)), "rank %d" % r


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_sum_reads_a_row_only_from_the_ranks_that_wrote_it(cuda_device, world):
    k, m = 64, 999
    rng = np.random.default_rng(7 + world)
    wrote = rng.random((world, m)) < 0.6
    wrote[:, 5] = False                                  # a row nobody wrote ends as zeros
    wrote[:, 6] = True
    host = []
    for r in range(world):
        h = rng.standard_normal((m, k)).astype(np.float32)
        h[~wrote[r]] = np.nan                            # must never be read
        host.append(h)
    words = (m + 31) // 32
    bitmaps = np.zeros((world, words), dtype=np.uint32)
    for r in range(world):
        rows = np.nonzero(wrote[r])[0]
        np.bitwise_or.at(bitmaps[r], rows >> 5, (np.uint32(1) << (rows & 31).astype(np.uint32)))
    d_maps = torch.from_numpy(bitmaps.view(np.int32).reshape(-1)).to(cuda_device)
    want = np.zeros((m, k), dtype=np.float32)
    for r in range(world):
        want += np.where(wrote[r][:, None], host[r], np.float32(0))

    bufs = [torch.from_numpy(h).to(cuda_device) for h in host]
    addrs = _addresses(bufs)
    for r in range(world):
        assert L.bidmat_b200_peer_allreduce_sum_rows(world, r, addrs, k, m, d_maps.data_ptr(), 7, None) == 0
    torch.cuda.synchronize()
    for r in range(world):
        got = bufs[r].cpu().numpy()
        assert not np.isnan(got).any()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "rank %d" % r
    assert not want[5].any()

    # the same in three row ranges, last range first: rows outside a range are left alone
    bufs = [torch.from_numpy(h).to(cuda_device) for h in host]
    addrs = _addresses(bufs)
    bounds = [0, 130, 131, m]
    for i in (2, 1, 0):
        for r in range(world):
            assert L.bidmat_b200_peer_allreduce_sum_rows_range(world, r, addrs, k, m, d_maps.data_ptr(), bounds[i],
                                                               bounds[i + 1], 3, None) == 0
        torch.cuda.synchronize()
        got = bufs[0].cpu().numpy()
        assert np.array_equal(got[bounds[i]:].view(np.uint32), want[bounds[i]:].view(np.uint32))
        if bounds[i] > 0:                                # not summed yet: still this rank's own partial
            assert np.array_equal(got[:bounds[i]].view(np.uint32), host[0][:bounds[i]].view(np.uint32))


def test_peer_sum_refuses_bad_arguments(cuda_device):
    a = torch.zeros(64, device=cuda_device)
    addrs = _addresses([a, a])
    assert L.bidmat_b200_peer_allreduce_sum(2, 2, addrs, 64, 0, None) == 1          # rank outside the world
    assert L.bidmat_b200_peer_allreduce_sum(2, 0, addrs, 62, 0, None) == 1          # not a multiple of 4 floats
    assert L.bidmat_b200_peer_allreduce_sum(1, 0, addrs, 64, 0, None) == 0          # one rank: nothing to add
    bad = (ctypes.c_ulonglong * 2)(a.data_ptr(), 0)
    assert L.bidmat_b200_peer_allreduce_sum(2, 0, bad, 64, 0, None) == 1            # a missing peer address
    three = _addresses([a, a, a])
    assert L.bidmat_b200_peer_allreduce_sum_rows(3, 0, three, 4, 16, a.data_ptr(), 0, None) == 1   # 2, 4 or 8 ranks
    assert L.bidmat_b200_mc_allreduce_sum(2, 0, None, 64, 0, None) == 1             # no multicast mapping
