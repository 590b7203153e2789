"""One rank's share of the sparse-dense path, on device-resident operands.

The sparse matrix is split by contiguous column ranges of (nearly) equal
nonzero count; the dense model A (k x m) is replicated; B, C and P follow the
columns.  A*S and DDS need no communication; the k x m result of B*^S is a
partial sum per rank and is summed over ranks with one allreduce
(the composition BIDMat leaves to its caller: GFunctions.ncclAllReduce,
src/main/scala/BIDMat/GFunctions.scala:175-203).

Shards carry local, zero-based column indices, as GSMat.colslice produces
(src/main/scala/BIDMat/GSMat.scala:77-104).
"""
import os

import torch

from . import _lib
from .gen import shard_columns

_L = _lib.lib


def _ck(err, what):
    if err != 0:
        raise RuntimeError("%s: %s" % (what, _lib.error_string(err)))


def slice_columns(jc, ir, data, col0, col1):
    """Columns [col0, col1) of a CSC matrix with re-based, zero-based column
    pointers (what GSMat.colslice produces).  Pure tensor slicing: works on CPU
    and CUDA tensors alike."""
    j0, j1 = int(jc[col0]), int(jc[col1])
    return (jc[col0:col1 + 1] - j0).to(torch.int32).contiguous(), ir[j0:j1].contiguous(), data[j0:j1].contiguous()


class ColumnShard:
    """Device tensors of one column range of a CSC matrix."""

    def __init__(self, m, jc, ir, data, col0, col1):
        self.m = int(m)
        self.col0, self.col1 = int(col0), int(col1)
        self.n = self.col1 - self.col0
        self.jc, self.ir, self.data = slice_columns(jc, ir, data, col0, col1)
        self.nnz = int(self.ir.numel())
        self.ic = torch.empty(self.nnz, dtype=torch.int32, device=ir.device)
        if self.nnz:
            _ck(_L.bidmat_b200_expand_jc(self.n, self.nnz, self.jc.data_ptr(), self.ic.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream), "expand_jc")


def make_shard(problem, rank, world):
    bounds = shard_columns(problem.jc, world)
    return ColumnShard(problem.m, problem.jc, problem.ir, problem.data, bounds[rank], bounds[rank + 1]), bounds


class PathStep:
    """A*S, DDS(A,B,S) and B*^S (+ allreduce) on one rank's shard, enqueued on
    one stream through the stream-ordered C ABI.

    B*^S goes through a prepared plan of the shard's structure (sorted once, here
    in the constructor) unless use_plan is False.  With a plan the product is
    written in overwrite mode: the rows of G that the shard names are overwritten
    every step and the others are never written, so G is not cleared between steps.
      * one GPU: G starts as zeros, its untouched rows stay zero;
      * several GPUs, peer-memory sum: every rank knows every rank's touched rows
        (bitmaps exchanged once) and reads a peer's row only when that peer wrote
        it, so what the untouched rows hold does not matter;
      * several GPUs, NCCL: NCCL adds whole buffers, so G is cleared every step.
    """

    def __init__(self, k, shard, A, B_local, stream, group=None, peer_reduce=False, use_plan=True, fuse=True):
        self.k, self.S, self.A, self.B, self.stream, self.group = int(k), shard, A, B_local, stream, group
        self.fuse = bool(fuse)      # A*S and DDS in one pass (run()); the separate calls stay available
        dev = A.device
        self.C = torch.zeros((shard.n, k), dtype=torch.float32, device=dev)
        self.P = torch.zeros(shard.nnz, dtype=torch.float32, device=dev)
        self.peer = None
        self.plan = None
        self.touched = None
        if use_plan and shard.nnz:
            from .mat import TransposedPlan
            self.plan = TransposedPlan(k, m=shard.m, ncols=shard.n, pir=shard.ir, pic=shard.ic)
        if group is not None and peer_reduce:
            # G lives in memory that the other GPUs of the box can address over NVLink;
            # the sum over ranks is then this library's own kernel, not a library collective.
            # If peer-addressable memory cannot be set up, NCCL sums the partials instead
            # (said on stderr; self.peer stays None).
            try:
                self._setup_peer_memory(shard, k, dev, group)
            except Exception as e:   # pragma: no cover - depends on the machine
                import sys
                print("bidmat_b200: peer-addressable memory unavailable (%s); summing B*^S partials with NCCL"
                      % (str(e).splitlines()[0] if str(e) else type(e).__name__), file=sys.stderr)
                self.peer = None
        if self.peer is None:
            self.G = torch.zeros((shard.m, k), dtype=torch.float32, device=dev)
        # A single-block plan (one rank's shard on many GPUs) can run in row ranges of equal work, the
        # sum of a range starting while the other ranges are still being multiplied.  The ranges run
        # from the last to the first: row popularity falls with the row index in the workloads this
        # path sees (words by frequency), so the last range holds nearly all the rows, i.e. nearly
        # all the bytes to sum, and its sum gets the longest head start.  The ranks agree on the
        # ranges once: the LARGEST of their bounds, so that a range summed after the local ranges
        # from it upwards are done is complete on every rank.  BIDMAT_B200_PIPE_PARTS=n turns it on.
        # Off by default.  Measured on 8 GPUs with the in-switch sum: B*^S and its sum alone take
        # 3.19 ms in 2 ranges against 3.84 ms in one piece, but the whole step 4.17 - 4.37 ms against
        # 4.03 ms: beside the sum's traffic the second range and A*S + DDS run that much slower, so
        # what the earlier start gains is lost again (3 ranges: 4.87 ms; peer loads/stores of the
        # touched rows in 4 ranges, first range first: 5.13 against 4.87 ms).
        self.mc = self.peer is not None and bool(self.peer["mc"])
        self.parts = None
        self._pending = None
        nparts = int(os.environ.get("BIDMAT_B200_PIPE_PARTS", "0"))
        if self.peer is not None and (self.touched is not None or self.mc) and nparts > 1:
            import ctypes
            import torch.distributed as dist
            bounds = (ctypes.c_int * (nparts + 1))()
            rc = _L.bidmat_b200_plan_row_parts(self.plan.handle, nparts, bounds)
            t = torch.tensor([0 if rc == 0 else 1] + [int(b) for b in bounds], dtype=torch.int64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)      # t[0] = 1 as soon as one rank cannot
            if int(t[0]) == 0:
                self.parts = [int(v) for v in t[1:]]
                self.parts[0], self.parts[-1] = 0, shard.m
        # clear G every step?  Not when the plan overwrites and nobody reads the untouched rows.
        self.overwrite = self.plan is not None and (group is None or (self.peer is not None and
                                                                     (self.touched is not None or self.mc)))

    def _setup_peer_memory(self, shard, k, dev, group):
        import ctypes
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        G = symm.empty((shard.m, k), dtype=torch.float32, device=dev)
        hdl = symm.rendezvous(G, group)
        world = dist.get_world_size(group)
        if world not in (2, 4, 8):
            raise RuntimeError("peer-memory sum supports 2, 4 or 8 GPUs")
        self.G = G
        self.peer = {
            "world": world, "rank": dist.get_rank(group), "handle": hdl,
            "addrs": (ctypes.c_ulonglong * world)(*[int(a) for a in hdl.buffer_ptrs]),
            "comm": torch.cuda.Stream(device=dev, priority=-1),
            "flag": torch.zeros(1, dtype=torch.float32, device=dev),
            "ctas": int(os.environ.get("BIDMAT_B200_PEER_CTAS", "0")),
            "mc": 0,
        }
        # A multicast mapping of the buffers (NVSwitch) lets the sum run inside the switch: half the
        # NVLink bytes per GPU.  Measured alone on 8 GPUs it takes 2.2 ms against 3.2 ms for peer
        # loads and stores of the touched rows (NCCL 2.5 ms), and since A*S and DDS share one pass
        # the sum is what the step waits for there: default from 4 GPUs up (BIDMAT_B200_PEER_MC=0/1
        # forces one or the other); on 2 GPUs the peer form hides completely and stays.
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        want_mc = os.environ.get("BIDMAT_B200_PEER_MC", "")
        use_mc = (world >= 4) if want_mc == "" else bool(int(want_mc))
        if mc and self.plan is not None and use_mc:
            self.peer["mc"] = mc
        self.G.zero_()
        if (self.plan is not None and k % 4 == 0 and not self.peer["mc"]
                and not int(os.environ.get("BIDMAT_B200_PEER_DENSE", "0"))):
            # every rank's touched-row bitmap, rank 0 first: exchanged once, the structure does not change
            mine = self.plan.touched_rows()
            allmaps = torch.empty(world * mine.numel(), dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(allmaps, mine, group=group)
            self.touched = allmaps
        torch.cuda.synchronize(dev)

    def touched_fraction(self):
        """Share of the m rows of G that this rank's shard names (None without a plan)."""
        if self.plan is None:
            return None
        return self.plan.info()["touched_rows"] / float(max(1, self.S.m))

    def dsmult(self):
        S = self.S
        with torch.cuda.stream(self.stream):
            self.C.zero_()   # GMat.GSMult clears the output before the native call (GMat.scala:1047)
            _ck(_L.bidmat_b200_dsmult_async(self.k, S.n, S.nnz, self.A.data_ptr(), S.data.data_ptr(), S.ir.data_ptr(),
                                            S.ic.data_ptr(), self.C.data_ptr(), self.stream.cuda_stream), "dsmult")

    def dds(self):
        S = self.S
        with torch.cuda.stream(self.stream):
            self.P.zero_()   # GSMat.DDS clears the values first (GSMat.scala:662)
            _ck(_L.bidmat_b200_dds_async(self.k, S.nnz, self.A.data_ptr(), self.B.data_ptr(), S.ir.data_ptr(),
                                         S.ic.data_ptr(), self.P.data_ptr(), self.stream.cuda_stream), "dds")

    def dsmult_dds(self):
        """C = A*S and P = DDS(A,B,S) in one pass over S (both gather the same columns of A)."""
        S = self.S
        with torch.cuda.stream(self.stream):
            self.C.zero_()
            self.P.zero_()
            _ck(_L.bidmat_b200_dsmult_dds_async(self.k, S.n, S.nnz, self.A.data_ptr(), self.B.data_ptr(),
                                                S.data.data_ptr(), S.ir.data_ptr(), S.ic.data_ptr(), self.C.data_ptr(),
                                                self.P.data_ptr(), self.stream.cuda_stream), "dsmult_dds")

    def dsmultT_local(self, data=None):
        """This rank's partial of B*^S over its column shard (no communication).
        `data`: other values on the same structure (e.g. a DDS result), default S's own."""
        S = self.S
        vals = S.data if data is None else data
        if self.parts is not None:
            return self._dsmultT_in_parts(vals)
        with torch.cuda.stream(self.stream):
            if not self.overwrite:
                self.G.zero_()   # GMat.GSMultT clears the output (GMat.scala:1082)
            if self.plan is not None:
                if self.mc:
                    # the switch adds whole buffers: rows this rank does not write must be zero
                    # (they hold the previous sum); the rows it writes are overwritten below
                    _ck(_L.bidmat_b200_plan_clear_untouched(self.plan.handle, self.k, self.G.data_ptr(),
                                                            self.stream.cuda_stream), "plan_clear_untouched")
                _ck(_L.bidmat_b200_dsmultT_planned(self.plan.handle, self.k, S.n, S.nnz, self.B.data_ptr(),
                                                   vals.data_ptr(), self.G.data_ptr(),
                                                   1 if self.overwrite else 0, self.stream.cuda_stream), "dsmultT (planned)")
            else:
                _ck(_L.bidmat_b200_dsmultT_async(self.k, S.n, S.nnz, self.B.data_ptr(), vals.data_ptr(),
                                                 S.ir.data_ptr(), S.ic.data_ptr(), self.G.data_ptr(), S.m,
                                                 self.stream.cuda_stream), "dsmultT")

    def _dsmultT_in_parts(self, vals):
        """B*^S range of rows after range of rows, last range first; the sum over the ranks of a
        range is queued on the side stream as soon as the range is done here (and, by the rank
        synchronisation in front of it, everywhere)."""
        import torch.distributed as dist
        S, pr = self.S, self.peer
        nparts = len(self.parts) - 1
        if self.mc:
            with torch.cuda.stream(self.stream):
                # the switch adds whole ranges: rows this rank does not write must be zero
                _ck(_L.bidmat_b200_plan_clear_untouched(self.plan.handle, self.k, self.G.data_ptr(),
                                                        self.stream.cuda_stream), "plan_clear_untouched")
        for r in reversed(range(nparts)):
            with torch.cuda.stream(self.stream):
                _ck(_L.bidmat_b200_dsmultT_planned_part(self.plan.handle, self.k, S.n, S.nnz, self.B.data_ptr(),
                                                        vals.data_ptr(), self.G.data_ptr(), 1, r,
                                                        self.stream.cuda_stream), "dsmultT (planned, part)")
                done = torch.cuda.Event()
                done.record(self.stream)
            with torch.cuda.stream(pr["comm"]):
                pr["comm"].wait_event(done)
                before = dist.all_reduce(pr["flag"], op=dist.ReduceOp.SUM, group=self.group, async_op=True)
                before.wait()
                if self.mc:
                    _ck(_L.bidmat_b200_mc_allreduce_sum_range(pr["world"], pr["rank"], pr["mc"], self.parts[r] * self.k,
                                                              (self.parts[r + 1] - self.parts[r]) * self.k, pr["ctas"],
                                                              pr["comm"].cuda_stream), "mc_allreduce_sum_range")
                else:
                    _ck(_L.bidmat_b200_peer_allreduce_sum_rows_range(pr["world"], pr["rank"], pr["addrs"], self.k, S.m,
                                                                     self.touched.data_ptr(), self.parts[r],
                                                                     self.parts[r + 1], pr["ctas"],
                                                                     pr["comm"].cuda_stream),
                        "peer_allreduce_sum_rows_range")
        with torch.cuda.stream(pr["comm"]):
            self._pending = dist.all_reduce(pr["flag"], op=dist.ReduceOp.SUM, group=self.group, async_op=True)

    def allreduce_start(self):
        """Starts the sum of the partials over ranks off the caller's stream, which
        is free to run A*S and DDS meanwhile; returns what to wait on."""
        if self.group is None:
            return None
        if self._pending is not None:         # the sums were queued range by range with the product
            work, self._pending = self._pending, None
            return work
        import torch.distributed as dist
        with torch.cuda.stream(self.stream):
            if self.peer is None:
                return dist.all_reduce(self.G, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            pr = self.peer
            # Rank synchronisation is a one-element NCCL allreduce before and after (it completes
            # on a rank only when every rank has reached it in stream order); the data moves in
            # this library's kernel over peer loads and stores.
            before = dist.all_reduce(pr["flag"], op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            with torch.cuda.stream(pr["comm"]):
                before.wait()
                if self.mc:
                    _ck(_L.bidmat_b200_mc_allreduce_sum(pr["world"], pr["rank"], pr["mc"], self.G.numel(), pr["ctas"],
                                                        pr["comm"].cuda_stream), "mc_allreduce_sum")
                elif self.touched is not None:
                    _ck(_L.bidmat_b200_peer_allreduce_sum_rows(pr["world"], pr["rank"], pr["addrs"], self.k, self.S.m,
                                                               self.touched.data_ptr(), pr["ctas"],
                                                               pr["comm"].cuda_stream), "peer_allreduce_sum_rows")
                else:
                    _ck(_L.bidmat_b200_peer_allreduce_sum(pr["world"], pr["rank"], pr["addrs"], self.G.numel(),
                                                          pr["ctas"], pr["comm"].cuda_stream), "peer_allreduce_sum")
                after = dist.all_reduce(pr["flag"], op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            return after

    def wait(self, work):
        if work is not None:
            with torch.cuda.stream(self.stream):
                work.wait()

    def dsmultT(self, data=None):
        self.dsmultT_local(data)
        self.wait(self.allreduce_start())

    def run(self):
        """One pass of the path.  The three operations are independent, so the
        transposed product goes first and its allreduce over NVLink overlaps
        A*S and DDS; the step ends when the reduced G is complete."""
        self.dsmultT_local()
        work = self.allreduce_start()
        if self.fuse:
            self.dsmult_dds()
        else:
            self.dsmult()
            self.dds()
        self.wait(work)

    def close(self):
        if self.plan is not None:
            self.plan.close()
            self.plan = None
