#!/usr/bin/env python
"""Benchmark of the sparse-dense path: A*S, DDS(A,B,S) and B*^S on the
LDA-shaped configuration (S 1e6 x 1e6, k = 256, Zipf rows, log-normal column
lengths), columns sharded over the GPUs of one box, the k x m result of B*^S
summed over ranks with one allreduce.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

A step is one pass of the three operations over the rank's shard.  Prints ONE
JSON line on rank 0.  Flops follow BIDMat's own convention, 2*k*nnz per
operation (Mat.nflops, src/main/scala/BIDMat/GMat.scala:1057,1092 and
GSMat.scala:665).

After the timed region the run checks its own results at full size, on the device
in fp64, on every rank: <A*S, B> = sum_j v_j * DDS_j = <B*^S, A> (the three
operations tied together by one scalar) and, on several GPUs, that every rank holds
bit-identical sums.  A failed check exits non-zero.

--impl reference times the CPU restatement of BIDMat's FMat/SMat loops
(oracle/) on the host cores instead; no CUDA kernel of this library runs on
that arm.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "nnz*k GFLOP/s over A*S + DDS + B*^S (2*k*nnz flops per operation)"
UNIT = "GFLOP/s"
FALLBACK_HBM_GBS = 6650.0
DRAM_PROFILE = os.path.join(ROOT, "profiles", "path_kernels_config2_quarter_dram.json")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the workload (debugging only)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--e2e-chunks", type=int, default=0, help="column chunks of the end-to-end pipeline (0: 8 per GPU "
                    "at one GPU, fewer per rank on several)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="target CPU time of the baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the sub-records timed outside the counted steps "
                    "(uniform-row DDS, unprepared B*^S, the reference's own CUDA kernels)")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--no-plan", action="store_true", help="B*^S through the reference-signature entry point "
                    "(sorts on every call) instead of the prepared plan")
    ap.add_argument("--no-fuse", action="store_true", help="A*S and DDS as two calls instead of the one-pass entry point")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="several GPUs: sum the B*^S partials with NCCL instead of the library's peer-memory kernel")
    ap.add_argument("--no-kernel-timing", action="store_true",
                    help="do not bracket the kernels with events inside the timed region (no roofline then)")
    ap.add_argument("--emulate-shard", default="", help="R/W: run rank R's shard of a W-way split on one GPU, "
                    "without communication (tuning aid; the JSON line then describes that shard only)")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed
    region runs (read-only queries)."""

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for name, bit in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------- helpers
def physical_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def algorithmic_bytes(op, k, nnz, n, m):
    """No-reuse gather model: every nonzero moves one k-vector of the dense
    operand plus its indices/values; the output is read and written once."""
    if op == "dsmult":
        return nnz * (4 * k + 12) + n * 8 * k
    if op == "dds":
        return nnz * (4 * k + 16) + n * 4 * k
    if op == "dsmultT":
        return nnz * (4 * k + 12) + m * 8 * k
    raise ValueError(op)


def compulsory_bytes(op, k, nnz, n, m, rows_touched, overwrite):
    if op == "dsmult_dds":  # one pass: the index lists and the named columns of A cross once for both results
        return 12 * nnz + 4 * k * rows_touched + 8 * k * n + 8 * nnz + 4 * k * n
    """What has to cross HBM at least once: the index and value lists, every dense
    column that is named once, and the output once (written) or twice (read and
    written, where the interface accumulates)."""
    if op == "dsmult":      # ir, ic, v; the named columns of A; C read + written (the ABI accumulates)
        return 12 * nnz + 4 * k * rows_touched + 8 * k * n
    if op == "dds":         # ir, ic; P read + written; named columns of A; B once
        return 16 * nnz + 4 * k * rows_touched + 4 * k * n
    if op == "dsmultT":     # values through the stored positions (position, value, write: 12) + sorted key, column, value (12);
        out = 4 * k * rows_touched * (1 if overwrite else 2)    # B once; named rows of G written (and read)
        return 24 * nnz + 4 * k * n + out
    raise ValueError(op)


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except Exception:
        pass
    return "unknown"


def load_oracle():
    """The CPU checker, switched to its -O3 -march=native build for timing (same bits
    as the plain build: tests/test_oracle.py)."""
    import oracle
    variant = oracle.use_native(True)
    return oracle, ("-O3 -march=native -ffp-contract=off" if variant == "native" else "-O2 -ffp-contract=off (plain x86-64)")


def cpu_sample_run(oracle, prob_host, threads):
    """Times the CPU restatement on a host-resident sample; returns per-op seconds."""
    A, B, jc, ir, data, m = prob_host
    out = {}
    t = time.perf_counter(); oracle.dsmult(A, data, ir, jc, nthreads=threads); out["dsmult"] = time.perf_counter() - t
    t = time.perf_counter(); oracle.dds(A, B, ir, jc, nthreads=threads); out["dds"] = time.perf_counter() - t
    t = time.perf_counter(); oracle.dsmultT(B, data, ir, jc, m, nthreads=threads); out["dsmultT"] = time.perf_counter() - t
    return out


def host_sample(problem, ncols):
    """First `ncols` columns of the workload, on the host: (A, B, jc, ir, data, m)."""
    ncols = max(1, min(ncols, problem.n))
    j1 = int(problem.jc[ncols])
    jc = problem.jc[:ncols + 1].cpu().numpy().astype(np.int32)
    ir = problem.ir[:j1].cpu().numpy()
    data = problem.data[:j1].cpu().numpy()
    if getattr(problem, "_A_host", None) is None:
        problem._A_host = problem.A.cpu().numpy()      # 1 GB at full size: copy once
    A = problem._A_host
    B = problem.B[:ncols].cpu().numpy()
    return (A, B, jc, ir, data, problem.m), j1


def calibrated_sample(oracle, problem, target_seconds, threads):
    """Picks a column count whose three CPU loops take about `target_seconds`:
    a probe of 20,000 columns gives the rate, one refinement corrects it."""
    avg = max(1.0, problem.nnz / problem.n)
    ncols = max(64, min(problem.n, 20000))
    for _ in range(2):
        sample, nnz = host_sample(problem, ncols)
        t = sum(cpu_sample_run(oracle, sample, threads).values())
        if ncols >= problem.n or 0.6 * target_seconds <= t <= 1.5 * target_seconds:
            break
        rate = max(nnz, 1) / max(t, 1e-6)             # nonzeros per second over the three loops
        ncols = int(max(64, min(problem.n, rate * target_seconds / avg)))
    return host_sample(problem, ncols) + (ncols,)


def generate(args, device):
    from bidmat_b200 import gen
    return gen.config2(args.scale, seed=args.seed, device=device)


def workload_config(problem, args, world, extra=None):
    # the same string in both arms and at every N (the line's "allreduce" key names the sum over the ranks)
    cfg = {"workload": "config2+4: LDA-shaped S %dx%d, nnz=%d, k=%d; ops A*S, DDS(A,B,S), B*^S"
                       % (problem.m, problem.n, problem.nnz, problem.k),
           "scale": args.scale, "seed": args.seed, "sharding": "columns by equal nnz, A replicated",
           "l2": "inputs larger than L2 (dense operands %.2f GB each)" % (4.0 * problem.k * problem.m / 1e9)}
    if extra:
        cfg.update(extra)
    return cfg


# --------------------------------------------------------------------------- reference arm
def run_reference(args, rank, world):
    if rank != 0:
        return
    dev = torch.device("cuda:0") if torch.cuda.is_available() else torch.device("cpu")
    scale = args.scale if dev.type == "cuda" else min(args.scale, 0.05)
    args.scale = scale
    problem = generate(args, dev)
    threads = os.cpu_count() or 1
    oracle, build = load_oracle()
    per_step = max(1.0, min(args.cpu_seconds, 150.0 / max(1, args.steps + args.warmup)))
    sample, nnz, ncols = calibrated_sample(oracle, problem, per_step, threads)
    k = problem.k
    for _ in range(args.warmup):
        cpu_sample_run(oracle, sample, threads)
    times = []
    per_op = {"dsmult": 0.0, "dds": 0.0, "dsmultT": 0.0}
    for _ in range(args.steps):
        r = cpu_sample_run(oracle, sample, threads)
        times.append(sum(r.values()))
        for o in per_op:
            per_op[o] += r[o]
    total = sum(times)
    value = 3 * 2.0 * k * nnz * args.steps / total / 1e9
    sample_txt = ("first %d columns (%d nonzeros, %.0f %% of the workload) per step, the same kind of sample as the "
                  "cpu_baseline of the b200 arm; B*^S threaded over k-ranges as FMat.maddT does (min(cores, k/32) "
                  "threads); checker built %s" % (ncols, nnz, 100.0 * nnz / max(1, problem.nnz), build))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "ms_per_step_note": "time of the column sample, not of the whole workload; value is a rate",
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(problem, args, 1, {"cpu_sample": sample_txt}),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample_txt, "cpu_model": cpu_model(),
                         "ops_gflops": {o: 2.0 * k * nnz * args.steps / per_op[o] / 1e9 for o in per_op}},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- verification
def checksum(t):
    """Two 64-bit checksums of a tensor's bits (plain and position-weighted sums of the
    32-bit words, wrapping), computed in slices to bound the temporaries."""
    bits = t.contiguous().view(torch.int32).flatten()
    c1 = torch.zeros((), dtype=torch.int64, device=t.device)
    c2 = torch.zeros((), dtype=torch.int64, device=t.device)
    step = 1 << 26
    for i in range(0, bits.numel(), step):
        b = bits[i:i + step].to(torch.int64)
        w = (torch.arange(i, i + b.numel(), device=t.device, dtype=torch.int64) % 8191) + 1
        c1 += b.sum()
        c2 += (b * w).sum()
    return torch.stack([c1, c2])


def dot64(x, y):
    """<x, y> in fp64 on the device, in slices."""
    x, y = x.flatten(), y.flatten()
    acc = torch.zeros((), dtype=torch.float64, device=x.device)
    step = 1 << 26
    for i in range(0, x.numel(), step):
        acc += (x[i:i + step].double() * y[i:i + step].double()).sum()
    return acc


def verify_step(st, problem, shard, B_local, world, dev):
    """Size-independent check of one completed step at the size it ran at."""
    import torch.distributed as dist
    t_c = dot64(st.C, B_local)
    t_p = dot64(st.P, shard.data)
    scale = dot64(st.P.abs(), shard.data.abs())
    t_g = dot64(st.G, problem.A)
    sums = torch.stack([t_c, t_p, scale])
    cs = checksum(st.G)
    ranks_identical = True
    tg_all = t_g.reshape(1)
    if world > 1:
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
        gathered = [torch.zeros_like(cs) for _ in range(world)]
        dist.all_gather(gathered, cs)
        ranks_identical = all(torch.equal(g, gathered[0]) for g in gathered)
        tg_list = [torch.zeros_like(tg_all) for _ in range(world)]
        dist.all_gather(tg_list, tg_all)
        tg_all = torch.cat(tg_list)
    t_c, t_p, scale = (float(v) for v in sums)
    err_c = abs(t_c - t_p) / max(scale, 1e-300)
    err_g = max(abs(float(v) - t_p) for v in tg_all) / max(scale, 1e-300)
    ok = bool(err_c <= 1e-5 and err_g <= 1e-4 and ranks_identical and np.isfinite(t_p) and scale > 0)
    return {"identity": bool(err_c <= 1e-5 and err_g <= 1e-4), "ranks_identical": bool(ranks_identical),
            "rel_err": max(err_c, err_g), "rel_err_AS_vs_DDS": err_c, "rel_err_BtS_vs_DDS": err_g,
            "tolerance": "1e-5 (A*S, DDS) and 1e-4 (B*^S) of sum|v_j P_j|", "ok": ok,
            "what": "<A*S,B> = sum v_j DDS_j = <B*^S,A> in fp64 on the device at the benchmark's size, all ranks; "
                    "64-bit checksums of G compared across ranks"}


# --------------------------------------------------------------------------- b200 arm
def run_b200(args, rank, local_rank, world):
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device for --impl b200 (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        opts = dist.ProcessGroupNCCL.Options()
        opts.is_high_priority_stream = True      # the allreduce shares the GPU with A*S and DDS
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
        group = dist.group.WORLD

    from bidmat_b200 import _lib, step as pstep
    L = _lib.lib

    problem = generate(args, dev)
    k, m = problem.k, problem.m
    if args.emulate_shard:
        er, ew = (int(x) for x in args.emulate_shard.split("/"))
        shard, bounds = pstep.make_shard(problem, er, ew)
    else:
        shard, bounds = pstep.make_shard(problem, rank, world)
    B_local = problem.B[shard.col0:shard.col1].contiguous()
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.synchronize()
    t_plan = time.perf_counter()
    st = pstep.PathStep(k, shard, problem.A, B_local, stream, group,
                        peer_reduce=(world > 1 and not args.nccl_allreduce), use_plan=not args.no_plan,
                        fuse=not args.no_fuse)
    fuse = st.fuse
    torch.cuda.synchronize()
    plan_ms = 1e3 * (time.perf_counter() - t_plan)
    plan_info = st.plan.info() if st.plan is not None else None

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ops = ("dsmultT", "dsmult_dds", "allreduce_exposed") if fuse else ("dsmultT", "dsmult", "dds", "allreduce_exposed")
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            st.run()
        barrier()
        L.bidmat_b200_timing_reset()
        L.bidmat_b200_timing_enable(0 if args.no_kernel_timing else 1)
        sampler = ClockSampler(physical_index(local_rank))
        launches0 = L.bidmat_b200_launch_count()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(ops) + 1)] for _ in range(args.steps)]
        sampler.start()
        barrier()
        t_start = torch.cuda.Event(enable_timing=True)
        t_end = torch.cuda.Event(enable_timing=True)
        t_start.record(stream)
        for s in range(args.steps):
            # same order as PathStep.run(): B*^S first, its allreduce overlaps A*S and DDS
            ev[s][0].record(stream)
            st.dsmultT_local(); ev[s][1].record(stream)
            work = st.allreduce_start()
            if fuse:
                st.dsmult_dds(); ev[s][2].record(stream)
            else:
                st.dsmult(); ev[s][2].record(stream)
                st.dds(); ev[s][3].record(stream)
            st.wait(work)
            ev[s][len(ops)].record(stream)
        t_end.record(stream)
        barrier()
        clocks = sampler.stop()
        launches = L.bidmat_b200_launch_count() - launches0
        L.bidmat_b200_timing_enable(0)
    total_ms = t_start.elapsed_time(t_end)
    op_ms = {o: sum(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(args.steps)) / args.steps
             for i, o in enumerate(ops)}
    kern = {}
    for label in ("dsmult_dds_chunk", "dsmult_ga_chunk", "dsmultT_ga_chunk", "dsmultT_permute", "dsmultT_rowsort", "ga_fixup", "dds_chunk",
                  "sort_hist", "sort_scan", "sort_scatter"):
        ms, cnt = _lib.timing_read(label)
        kern[label] = {"launches_per_step": cnt / args.steps, "avg_ms": ms / cnt if cnt else None,
                       "ms_per_step": ms / args.steps}
    L.bidmat_b200_timing_reset()

    # the step's own results, checked at this size on every rank (outside the timed region)
    verified = None
    if not args.no_verify and not args.emulate_shard:
        verified = verify_step(st, problem, shard, B_local, world, dev)

    # the sum of the partials alone, with nothing running beside it (several GPUs; after the check above,
    # the buffers then hold sums of sums)
    sum_alone_ms = None
    if world > 1 and not args.emulate_shard:
        with torch.cuda.stream(stream):
            def sum_only():
                st.wait(st.allreduce_start())
            sum_alone_ms = time_calls(sum_only, stream, 3, 1)

    # max over ranks
    red = torch.tensor([total_ms] + [op_ms[o] for o in ops], dtype=torch.float64, device=dev)
    nnz_all = torch.tensor([shard.nnz], dtype=torch.float64, device=dev)
    touched = torch.tensor([st.touched_fraction() or 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(red, op=dist.ReduceOp.MAX)
        dist.all_reduce(nnz_all, op=dist.ReduceOp.SUM)
        dist.all_reduce(touched, op=dist.ReduceOp.SUM)
    total_ms = float(red[0])
    op_ms_max = {o: float(red[1 + i]) for i, o in enumerate(ops)}
    nnz_total = int(nnz_all[0])
    ms_per_step = total_ms / args.steps
    value = 3 * 2.0 * k * nnz_total / (ms_per_step * 1e-3) / 1e9
    overwrite = bool(st.overwrite)
    allreduce_kind = (None if world == 1 else
                      ("library kernel through the NVSwitch (multimem.ld_reduce / multimem.st)" if st.mc else
                       "library kernel over NVLink peer memory, touched rows only" if st.touched is not None
                       else "library kernel over NVLink peer memory") if st.peer is not None else "NCCL")

    st_parts = st.parts
    extras = None
    if rank == 0 and world == 1 and not args.no_extras and not args.emulate_shard:
        extras = run_extras(args, problem, shard, B_local, st, dev, stream)
    st_rows_touched = plan_info["touched_rows"] if plan_info else None

    # ----- end to end through the operator interface with host buffers (rank-local shard)
    e2e = None
    if not args.no_e2e and not args.emulate_shard:
        st.close()
        del st
        torch.cuda.empty_cache()
        e2e = run_e2e(args, problem, shard, B_local, dev, rank, world, group)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    dram = load_dram_profile()
    roof_ops = {}
    op_list = ((("dsmult_dds", "dsmult_dds_chunk", ("dsmult", "dds")),) if fuse else
               (("dsmult", "dsmult_ga_chunk", ("dsmult",)), ("dds", "dds_chunk", ("dds",)))) + \
              (("dsmultT", "dsmultT_ga_chunk", ("dsmultT",)),)
    for o, label, parts in op_list:
        # algorithmic bytes of the rank's whole shard (for the one-pass kernel: of both operations it
        # computes); the launches of one step together process it once
        ab = sum(algorithmic_bytes(q, k, shard.nnz, shard.n, m) for q in parts)
        ms = kern[label]["ms_per_step"]
        if o == "dsmultT" and world > 1:
            op_ms_max[o] += op_ms_max["allreduce_exposed"]   # the part of the allreduce that A*S and DDS did not hide
        rec = {"kernel": label, "kernel_ms": ms, "launches_per_step": kern[label]["launches_per_step"],
               "operations": list(parts), "algorithmic_bytes": ab,
               "achieved_gbs": ab / (ms * 1e-3) / 1e9 if ms else None,
               "frac": ab / (ms * 1e-3) / 1e9 / peak if ms else None,
               "op_ms_max_over_ranks": op_ms_max[o],
               "op_frac": ab / (op_ms_max[o] * 1e-3) / 1e9 / peak,
               "op_gflops": len(parts) * 2.0 * k * nnz_total / (op_ms_max[o] * 1e-3) / 1e9}
        if st_rows_touched is not None:
            cb = compulsory_bytes(o, k, shard.nnz, shard.n, m, st_rows_touched, overwrite and o == "dsmultT")
            rec["compulsory_bytes"] = cb
            rec["compulsory_frac"] = cb / (ms * 1e-3) / 1e9 / peak if ms else None
        d = dram.get(o) if dram else None
        if d and ms and world == 1:
            # DRAM bytes per nonzero from the quarter-size ncu capture, scaled by this run's nonzeros; the
            # output traffic of B*^S grows with the number of (column block, row) runs instead
            db = d["dram_bytes_per_nnz"] * shard.nnz
            if o == "dsmultT" and plan_info and "dram_bytes_per_row_run" in d:
                db += d["dram_bytes_per_row_run"] * plan_info["row_runs"]
                if overwrite:
                    db -= d.get("overwrite_saves_bytes_per_touched_row", 0) * plan_info["touched_rows"]
            rec["dram_bytes"] = db
            rec["dram_frac"] = db / (ms * 1e-3) / 1e9 / peak
            rec["l2_frac"] = d.get("lts_throughput_frac")
        roof_ops[o] = rec
    dom = max(roof_ops, key=lambda o: roof_ops[o]["kernel_ms"] or 0.0)
    roofline = {"bound": "hbm", "kernel": roof_ops[dom]["kernel"], "op": dom,
                "achieved": roof_ops[dom]["achieved_gbs"], "peak": peak, "unit": "GB/s",
                "frac": roof_ops[dom]["frac"], "peak_source": peak_src,
                "traffic": roof_ops[dom].get("dram_bytes"),
                "traffic_note": ("DRAM bytes per step of this operation's gather kernels: bytes per nonzero from an ncu "
                                 "capture of the quarter-size workload (%s, build %s) times this run's nonzeros"
                                 % (os.path.relpath(DRAM_PROFILE, ROOT), dram.get("build", "?")) if dram else
                                 "no committed capture for this build"),
                "frac_note": "algorithmic bytes are the no-reuse gather model (every nonzero moves a k-vector); hot rows "
                             "are served by L2, so frac can exceed 1: dram_frac (measured DRAM bytes / time / peak) and "
                             "compulsory_frac (bytes that must cross HBM at least once / time / peak) bracket the truth",
                "ops": roof_ops, "kernels": kern}
    if extras and extras.get("uniform_dds"):
        roofline["hbm_bound_case"] = extras["uniform_dds"]

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(problem, args, world, {
            "dsmult_dds_path": ("one pass over S for A*S and DDS (bidmat_b200_dsmult_dds_async): the gather of A's "
                                "columns is shared" if fuse else "two calls (dsmult, dds)"),
            "dsmultT_path": ("reference-signature entry point (sorts every call)" if args.no_plan else
                             "prepared plan: structure sorted once outside the timed region (%.0f ms together with "
                             "the step's buffers, %s bytes held), values read through the stored positions on "
                             "every call, %s" % (plan_ms, plan_info["bytes"] if plan_info else "?",
                                                                "overwrite mode (G not cleared between steps)"
                                                                if overwrite else "G cleared every step"))}),
        "clocks": clocks, "gpu_launches": int(launches), "roofline": roofline, "e2e": e2e, "verified": verified,
        "allreduce_exposed_ms": op_ms_max["allreduce_exposed"] if world > 1 else 0.0,
        "allreduce": allreduce_kind, "allreduce_alone_ms_rank0": sum_alone_ms,
        "dsmultT_row_parts": (len(st_parts) - 1) if st_parts else None,
        "touched_row_fraction_mean_over_ranks": float(touched[0]) / world if plan_info else None,
        "plan": plan_info,
    }
    if extras:
        line["extras"] = {k_: v for k_, v in extras.items() if k_ != "uniform_dds"}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args, problem)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    bad = (verified is not None and not verified["ok"]) or (e2e is not None and e2e.get("verified") is False)
    if bad:
        sys.stderr.write("bench.py: result verification FAILED: %s\n" % json.dumps({"step": verified, "e2e": e2e}))
        sys.exit(3)


def load_dram_profile():
    try:
        with open(DRAM_PROFILE) as f:
            return json.load(f)
    except Exception:
        return None


def time_calls(fn, stream, reps, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        fn()
        b.record(stream)
        b.synchronize()
        out.append(a.elapsed_time(b))
    return statistics.median(out)


def run_extras(args, problem, shard, B_local, st, dev, stream):
    """Sub-records timed outside the counted steps (one GPU)."""
    from bidmat_b200 import _lib, gen, step as pstep
    L = _lib.lib
    peak, _ = measured_peak()
    out = {}
    k, m = problem.k, problem.m
    with torch.cuda.stream(stream):
        # (1) B*^S through the reference-signature entry point: sorts on every call
        G2 = torch.zeros((m, k), dtype=torch.float32, device=dev)

        def dropin():
            G2.zero_()
            err = L.bidmat_b200_dsmultT_async(k, shard.n, shard.nnz, B_local.data_ptr(), shard.data.data_ptr(),
                                              shard.ir.data_ptr(), shard.ic.data_ptr(), G2.data_ptr(), m,
                                              stream.cuda_stream)
            assert err == 0, _lib.error_string(err)
        out["dsmultT_unprepared_ms"] = time_calls(dropin, stream, 3, 1)

        # (1a) the synchronous native of the reference (no stream, no m, no handle) with plans kept by the
        # library: fingerprint of the structure on every call, plan built at the second sighting
        def dropin_kept():
            G2.zero_()
            torch.cuda.synchronize(dev)
            err = L.bidmat_b200_dsmultT(k, shard.n, shard.nnz, B_local.data_ptr(), shard.data.data_ptr(),
                                        shard.ir.data_ptr(), shard.ic.data_ptr(), G2.data_ptr())
            assert err == 0, _lib.error_string(err)
        L.bidmat_b200_set_auto_plan(1)
        try:
            out["dsmultT_reference_signature_kept_plan_ms"] = time_calls(dropin_kept, stream, 3, 2)
            import ctypes
            info = (ctypes.c_longlong * 6)()
            L.bidmat_b200_auto_plan_info(info, 6)
            out["kept_plan_info"] = {"built": int(info[1]), "planned_calls": int(info[2]), "plain_calls": int(info[3])}
        finally:
            L.bidmat_b200_set_auto_plan(0)
        del G2
        # (1b) A*S and DDS as two calls (what the one-pass entry point replaces)
        out["dsmult_alone_ms"] = time_calls(st.dsmult, stream, 3, 1)
        out["dds_alone_ms"] = time_calls(st.dds, stream, 3, 1)

    # (2) the reference's own CUDA kernels on the same operands, and an element-wise comparison at full size
    try:
        import oracle
        if oracle.ref_gpu_available():
            out["reference_gpu"] = reference_gpu_record(oracle, problem, shard, B_local, st, dev, stream)
    except Exception as e:          # the comparison is an extra: report, do not fail the run
        out["reference_gpu"] = {"unavailable": "%s: %s" % (type(e).__name__, str(e).splitlines()[0] if str(e) else "")}

    # (3) the HBM-bound case: DDS on uniform rows (config 3), where every gather is a DRAM read
    try:
        recs = []
        for kk in (256, 512):
            p3 = gen.config3(kk, args.scale, args.seed, dev)
            sh3, _ = pstep.make_shard(p3, 0, 1)
            P3 = torch.zeros(sh3.nnz, dtype=torch.float32, device=dev)
            with torch.cuda.stream(stream):
                def dds3():
                    err = L.bidmat_b200_dds_async(kk, sh3.nnz, p3.A.data_ptr(), p3.B.data_ptr(), sh3.ir.data_ptr(),
                                                  sh3.ic.data_ptr(), P3.data_ptr(), stream.cuda_stream)
                    assert err == 0
                ms = time_calls(dds3, stream, 5, 2)
            ab = algorithmic_bytes("dds", kk, sh3.nnz, sh3.n, p3.m)
            recs.append({"workload": "config3: S %dx%d uniform rows, 64 per column, nnz=%d, k=%d; DDS"
                                     % (p3.m, p3.n, sh3.nnz, kk),
                         "ms": ms, "algorithmic_bytes": ab, "achieved_gbs": ab / (ms * 1e-3) / 1e9,
                         "frac": ab / (ms * 1e-3) / 1e9 / peak,
                         "gflops": 2.0 * kk * sh3.nnz / (ms * 1e-3) / 1e9})
            del p3, sh3, P3
            torch.cuda.empty_cache()
        out["uniform_dds"] = {"note": "rows uniform over 5e5 (A is %d x L2 at k=512): the no-reuse model is the DRAM "
                                      "traffic here, so frac is a true fraction of the HBM roofline; timed outside "
                                      "the counted steps, median of 5" % 8, "cases": recs}
    except Exception as e:
        out["uniform_dds"] = {"unavailable": "%s: %s" % (type(e).__name__, str(e).splitlines()[0] if str(e) else "")}
    return out


def reference_gpu_record(oracle, problem, shard, B_local, st, dev, stream):
    """BIDMat's own dsmult / dsmultT / dds (jni/src/Arith.cu) compiled for sm_100a, run
    once each on this workload's operands, timed on the host around the (synchronous)
    launchers; results compared element by element with this library's, relative to
    sum|terms| computed by this library on absolute values."""
    from bidmat_b200 import _lib
    L = _lib.lib
    k, m = problem.k, problem.m
    torch.cuda.synchronize()
    rec = {"source": "reference's jni/src/Arith.cu compiled for sm_100a (oracle/_ref/libarith_ref.so); float atomics"}
    ptr = lambda t: t.data_ptr()

    def scaled_err(mine, ref, absop):
        scale = absop()
        err = (mine.double() - ref.double()).abs()
        worst = float((err / (scale.double() + 1e-30)).max())
        del scale, err
        return worst

    def timed(fn):
        torch.cuda.synchronize()
        t = time.perf_counter(); fn(); torch.cuda.synchronize()
        return 1e3 * (time.perf_counter() - t)

    with torch.cuda.stream(stream):
        absd = shard.data.abs()
        # A*S
        ref = torch.zeros_like(st.C)
        rec["dsmult_ms"] = timed(lambda: oracle.ref_gpu_dsmult(k, shard.n, shard.nnz, ptr(problem.A), ptr(shard.data),
                                                               ptr(shard.ir), ptr(shard.ic), ptr(ref)))
        st.dsmult(); torch.cuda.synchronize()

        def abs_as():
            out = torch.zeros_like(st.C)
            Aabs = problem.A.abs()
            assert L.bidmat_b200_dsmult_async(k, shard.n, shard.nnz, ptr(Aabs), ptr(absd), ptr(shard.ir),
                                              ptr(shard.ic), ptr(out), stream.cuda_stream) == 0
            torch.cuda.synchronize()
            return out
        rec["dsmult_max_err_over_sum_abs_terms"] = scaled_err(st.C, ref, abs_as)
        del ref
        # DDS
        ref = torch.zeros_like(st.P)
        rec["dds_ms"] = timed(lambda: oracle.ref_gpu_dds(k, shard.nnz, ptr(problem.A), ptr(B_local), ptr(shard.ir),
                                                         ptr(shard.ic), ptr(ref)))
        st.dds(); torch.cuda.synchronize()

        def abs_dds():
            out = torch.zeros_like(st.P)
            Aabs, Babs = problem.A.abs(), B_local.abs()
            assert L.bidmat_b200_dds_async(k, shard.nnz, ptr(Aabs), ptr(Babs), ptr(shard.ir), ptr(shard.ic), ptr(out),
                                           stream.cuda_stream) == 0
            torch.cuda.synchronize()
            return out
        rec["dds_max_err_over_sum_abs_terms"] = scaled_err(st.P, ref, abs_dds)
        del ref
        # B*^S
        ref = torch.zeros((m, k), dtype=torch.float32, device=dev)
        rec["dsmultT_ms"] = timed(lambda: oracle.ref_gpu_dsmultT(k, shard.n, shard.nnz, ptr(B_local), ptr(shard.data),
                                                                 ptr(shard.ir), ptr(shard.ic), ptr(ref)))
        st.dsmultT_local(); torch.cuda.synchronize()

        def abs_t():
            out = torch.zeros((m, k), dtype=torch.float32, device=dev)
            Babs = B_local.abs()
            assert L.bidmat_b200_dsmultT_async(k, shard.n, shard.nnz, ptr(Babs), ptr(absd), ptr(shard.ir),
                                               ptr(shard.ic), ptr(out), m, stream.cuda_stream) == 0
            torch.cuda.synchronize()
            return out
        rec["dsmultT_max_err_over_sum_abs_terms"] = scaled_err(st.G, ref, abs_t)
        del ref
    rec["within_tolerance"] = bool(rec["dsmult_max_err_over_sum_abs_terms"] <= 1e-5 and
                                   rec["dds_max_err_over_sum_abs_terms"] <= 1e-5 and
                                   rec["dsmultT_max_err_over_sum_abs_terms"] <= 1e-4)
    rec["step_ms"] = rec["dsmult_ms"] + rec["dds_ms"] + rec["dsmultT_ms"]
    rec["gflops"] = 3 * 2.0 * k * shard.nnz / (rec["step_ms"] * 1e-3) / 1e9
    torch.cuda.empty_cache()
    return rec


def pcie_bandwidth(dev):
    """Pinned-memory copy bandwidth in both directions, one 1 GB copy each (GB/s)."""
    nbytes = 1 << 30
    h = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    out = {}
    for name, (src, dst) in (("h2d", (h, d)), ("d2h", (d, h))):
        dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); dst.copy_(src, non_blocking=True); b.record(); b.synchronize()
        out[name] = nbytes / (a.elapsed_time(b) * 1e-3) / 1e9
    del h, d
    return out


def run_e2e(args, problem, shard, B_local, dev, rank, world, group):
    """The three operations through the GMat / GSMat operator interface with HOST
    operands, host-to-device and device-to-host copies inside the timed region.

    The shard is cut into column chunks (GSMat.colslice semantics).  Per step: the
    model A is uploaded (one GPU: whole; several: every rank uploads 1/N of it and the
    ranks all-gather it over NVLink); then chunk after chunk S and B are uploaded on a
    copy stream while the previous chunk computes C = A*S, P = DDS(A,B,S) and
    G += B *^ S through the operators, and each chunk's C and P go back to the host on
    a second copy stream as soon as they exist.  G is complete after the last chunk
    (summed over ranks on several GPUs; every rank then downloads 1/N of it)."""
    import torch.distributed as dist
    from bidmat_b200 import gen
    from bidmat_b200.mat import GMat, GSMat, DDS
    k, m = problem.k, problem.m
    nchunks = args.e2e_chunks or (8 if world == 1 else max(2, 8 // world))
    pcie = pcie_bandwidth(dev)

    # ---- host operands (pinned), prepared once: they are the inputs of every step
    pin = lambda t: t.cpu().pin_memory()
    # Column chunks of equal nonzero count, except that the last regular chunk is cut 3 : 1 again:
    # what is multiplied after the last upload has arrived delays the download of G, so the
    # last chunk is a small one.
    if nchunks >= 2:
        fr = [i / float(nchunks) for i in range(nchunks)] + [(nchunks - 0.25) / nchunks, 1.0]
        targets = torch.tensor([int(shard.nnz * f) for f in fr[1:-1]], dtype=shard.jc.dtype, device=shard.jc.device)
        cuts = torch.searchsorted(shard.jc.contiguous(), targets).clamp_(0, shard.n).tolist()
        cb = [0] + [int(c) for c in cuts] + [shard.n]
        for i in range(1, len(cb)):
            cb[i] = max(cb[i], cb[i - 1])
    else:
        cb = gen.shard_columns(shard.jc, nchunks)
    chunks = []
    for c in range(len(cb) - 1):
        c0, c1 = cb[c], cb[c + 1]
        j0, j1 = int(shard.jc[c0]), int(shard.jc[c1])
        if c1 <= c0:
            continue
        chunks.append({"c0": c0, "c1": c1, "j0": j0, "j1": j1,
                       "jc": pin((shard.jc[c0:c1 + 1] - j0).to(torch.int32)), "ir": pin(shard.ir[j0:j1]),
                       "data": pin(shard.data[j0:j1]), "B": pin(B_local[c0:c1])})
    a0, a1 = (m * rank) // world, (m * (rank + 1)) // world          # this rank's rows of A (and of the reduced G)
    hA = pin(problem.A[a0:a1])
    hC = torch.empty((shard.n, k), dtype=torch.float32).pin_memory()
    hP = torch.empty(shard.nnz, dtype=torch.float32).pin_memory()
    hG = torch.empty((a1 - a0, k), dtype=torch.float32).pin_memory()
    h2d = hA.numel() * 4 + sum(sum(ch[x].numel() * ch[x].element_size() for x in ("jc", "ir", "data", "B")) for ch in chunks)
    d2h = (hC.numel() + hP.numel() + hG.numel()) * 4

    up = torch.cuda.Stream(device=dev)      # host -> device copies
    down = torch.cuda.Stream(device=dev)    # device -> host copies
    main = torch.cuda.current_stream(dev)
    d_A = torch.empty((m, k), dtype=torch.float32, device=dev)
    d_Ain = d_A[a0:a1] if world == 1 else torch.empty((a1 - a0, k), dtype=torch.float32, device=dev)
    G = GMat(torch.empty((m, k), dtype=torch.float32, device=dev))

    phases = {}

    def one():
        evs = []
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        marks[0].record(main)
        with torch.cuda.stream(up):
            d_Ain.copy_(hA, non_blocking=True)
            ev_a = torch.cuda.Event(); ev_a.record(up)
            dchunks = []
            for ch in chunks:
                dchunks.append({x: ch[x].to(dev, non_blocking=True) for x in ("jc", "ir", "data", "B")})
                e = torch.cuda.Event(); e.record(up); evs.append(e)
        main.wait_event(ev_a)
        if group is not None:
            dist.all_gather_into_tensor(d_A, d_Ain, group=group)     # the model reaches every GPU over NVLink
        A = GMat(d_A)
        marks[1].record(main)                           # the whole model is on the device
        G.clear()
        for ch, dch, e in zip(chunks, dchunks, evs):
            main.wait_event(e)
            S = GSMat.from_csc(m, ch["c1"] - ch["c0"], dch["jc"], dch["ir"], dch["data"])
            B = GMat(dch["B"])
            if args.no_fuse:
                C = A * S                               # complete on return, like the BIDMat call
            else:
                C, P = A.GSMultDDS(B, S)                # A*S and DDS(A,B,S) in one pass over S
            done = torch.cuda.Event(); done.record(main)
            with torch.cuda.stream(down):
                down.wait_event(done)
                hC[ch["c0"]:ch["c1"]].copy_(C.t, non_blocking=True)
                C.t.record_stream(down)                 # the copy outlives this chunk's Python objects
            if args.no_fuse:
                P = DDS(A, B, S)
                done = torch.cuda.Event(); done.record(main)
            with torch.cuda.stream(down):
                down.wait_event(done)
                hP[ch["j0"]:ch["j1"]].copy_(P.pdata, non_blocking=True)
                P.pdata.record_stream(down)
            B.maddT(S, G)                               # G += B *^ S
        marks[2].record(main)                           # all chunks multiplied
        if group is not None:
            dist.all_reduce(G.t, op=dist.ReduceOp.SUM, group=group)
        marks[3].record(main)                           # G summed over the ranks
        with torch.cuda.stream(down):
            down.wait_event(marks[3])
            hG.copy_(G.t[a0:a1], non_blocking=True)
            marks[4].record(down)                       # everything is back on the host
        torch.cuda.synchronize()
        for i, name in enumerate(("model_upload_and_allgather", "chunks", "allreduce", "last_downloads")):
            phases[name] = marks[i].elapsed_time(marks[i + 1])

    one()  # warm-up (allocator, scratch pool)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.e2e_steps):
        one()
    t1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([t0.elapsed_time(t1) / args.e2e_steps], dtype=torch.float64, device=dev)
    nnz = torch.tensor([shard.nnz], dtype=torch.float64, device=dev)
    bytes_ = torch.tensor([h2d, d2h], dtype=torch.float64, device=dev)
    # the host results of the last step, tied together like the device results
    hB = torch.cat([ch["B"] for ch in chunks]).numpy()
    hdata = torch.cat([ch["data"] for ch in chunks]).numpy()
    sums = torch.tensor([np.dot(hC.numpy().reshape(-1).astype(np.float64), hB.reshape(-1).astype(np.float64)),
                         np.dot(hP.numpy().astype(np.float64), hdata.astype(np.float64)),
                         np.dot(np.abs(hP.numpy()).astype(np.float64), np.abs(hdata).astype(np.float64)),
                         np.dot(hG.numpy().reshape(-1).astype(np.float64),
                                hA.numpy().reshape(-1).astype(np.float64))], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(nnz, op=dist.ReduceOp.SUM)
        dist.all_reduce(bytes_, op=dist.ReduceOp.SUM)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    t_c, t_p, scale, t_g = (float(v) for v in sums)
    rel = max(abs(t_c - t_p) / max(scale, 1e-300) / 1e-5, abs(t_g - t_p) / max(scale, 1e-300) / 1e-4)
    bound_ms = max(float(bytes_[0]) / world / (pcie["h2d"] * 1e9), float(bytes_[1]) / world / (pcie["d2h"] * 1e9)) * 1e3
    return {"value": 3 * 2.0 * k * float(nnz[0]) / (float(ms[0]) * 1e-3) / 1e9, "unit": UNIT,
            "ms_per_step": float(ms[0]), "steps": args.e2e_steps,
            "h2d_bytes_per_step": int(bytes_[0]), "d2h_bytes_per_step": int(bytes_[1]),
            "pcie_gbs": pcie, "pcie_bound_ms": bound_ms, "ms_over_pcie_bound": float(ms[0]) / bound_ms,
            "chunks_per_rank": len(chunks), "phases_ms_rank0_last_step": phases,
            "verified": bool(rel <= 1.0 and np.isfinite(rel)),
            "verified_rel_err_over_tolerance": rel,
            "api": ("GMat * GSMat, DDS(GMat, GMat, GSMat)" if args.no_fuse else "GMat.GSMultDDS(GMat, GSMat)") +
                   ", GMat.maddT(GSMat) per column chunk with pinned host operands; "
                   "uploads and downloads on their own streams, overlapped with the products"}


def cpu_baseline(args, problem):
    threads = os.cpu_count() or 1
    oracle, build = load_oracle()
    sample, nnz, ncols = calibrated_sample(oracle, problem, args.cpu_seconds, threads)
    r = cpu_sample_run(oracle, sample, threads)
    k = problem.k
    total = sum(r.values())
    out = {"value": 3 * 2.0 * k * nnz / total / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
           "sample": "first %d columns (%d nonzeros) of the workload, each loop once; B*^S threaded over k-ranges "
                     "as FMat.maddT does (min(cores, k/32) threads); checker built %s" % (ncols, nnz, build),
           "cpu_model": cpu_model(), "seconds": total,
           "ops_gflops": {o: 2.0 * k * nnz / r[o] / 1e9 for o in r}}
    try:
        if oracle.ref_available():
            A, B, jc, ir, data, m = sample
            t = time.perf_counter(); oracle.ref_smcscm(A, data, ir, jc); dt = time.perf_counter() - t
            out["reference_build_smcscm_gflops"] = 2.0 * k * nnz / dt / 1e9
    except Exception as e:  # the cross-check is optional
        out["reference_build_smcscm_gflops"] = "unavailable: %s" % e
    return out


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        # launched without torchrun: re-launch one process per GPU
        port = 29500 + (os.getpid() % 2000)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.gpus),
               "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    run_b200(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
