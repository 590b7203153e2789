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

# dram__bytes_read.sum + dram__bytes_write.sum per step from a one-pass ncu capture of the
# default workload (seed 0, full size, one GPU); the capture's summary is committed under profiles/.
# Reported only when the run is that workload.
MEASURED_DRAM_TRAFFIC = {"dsmult": 31.25e9, "dds": 30.50e9, "dsmultT": 31.75e9}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the workload (debugging only)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="target CPU time of the baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
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
            self._stop.wait(0.1)

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


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except Exception:
        pass
    return "unknown"


def cpu_sample_run(prob_host, threads, repeats=1):
    """Times the CPU restatement on a host-resident sample; returns per-op seconds."""
    import oracle
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


def calibrated_sample(problem, target_seconds, threads):
    """Picks a column count whose three CPU loops take about `target_seconds`:
    a probe of 20,000 columns gives the rate, one refinement corrects it."""
    avg = max(1.0, problem.nnz / problem.n)
    ncols = max(64, min(problem.n, 20000))
    for _ in range(2):
        sample, nnz = host_sample(problem, ncols)
        t = sum(cpu_sample_run(sample, threads).values())
        if ncols >= problem.n or 0.6 * target_seconds <= t <= 1.5 * target_seconds:
            break
        rate = max(nnz, 1) / max(t, 1e-6)             # nonzeros per second over the three loops
        ncols = int(max(64, min(problem.n, rate * target_seconds / avg)))
    return host_sample(problem, ncols) + (ncols,)


def generate(args, device):
    from bidmat_b200 import gen
    return gen.config2(args.scale, seed=args.seed, device=device)


# --------------------------------------------------------------------------- reference arm
def run_reference(args, rank, world):
    if rank != 0:
        return
    dev = torch.device("cuda:0") if torch.cuda.is_available() else torch.device("cpu")
    scale = args.scale if dev.type == "cuda" else min(args.scale, 0.05)
    args.scale = scale
    problem = generate(args, dev)
    threads = os.cpu_count() or 1
    per_step = max(1.0, min(args.cpu_seconds, 150.0 / max(1, args.steps + args.warmup)))
    sample, nnz, ncols = calibrated_sample(problem, per_step, threads)
    k = problem.k
    for _ in range(args.warmup):
        cpu_sample_run(sample, threads)
    times = []
    per_op = {"dsmult": 0.0, "dds": 0.0, "dsmultT": 0.0}
    for _ in range(args.steps):
        r = cpu_sample_run(sample, threads)
        times.append(sum(r.values()))
        for o in per_op:
            per_op[o] += r[o]
    total = sum(times)
    value = 3 * 2.0 * k * nnz * args.steps / total / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(problem, args, 1),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "first %d columns (%d nonzeros) of the workload per step; B*^S threaded over "
                                   "k-ranges as FMat.maddT does (min(cores, k/32) threads)" % (ncols, nnz),
                         "cpu_model": cpu_model(),
                         "ops_gflops": {o: 2.0 * k * nnz * args.steps / per_op[o] / 1e9 for o in per_op}},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(problem, args, world):
    return {"workload": "config2+4: LDA-shaped S %dx%d, nnz=%d, k=%d; ops A*S, DDS(A,B,S), B*^S%s"
                        % (problem.m, problem.n, problem.nnz, problem.k, " + allreduce" if world > 1 else ""),
            "scale": args.scale, "seed": args.seed, "sharding": "columns by equal nnz, A replicated",
            "l2": "inputs larger than L2 (dense operands %.2f GB each)" % (4.0 * problem.k * problem.m / 1e9)}


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
    from bidmat_b200.mat import GMat, GSMat, SMat, DDS
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
    st = pstep.PathStep(k, shard, problem.A, B_local, stream, group, peer_reduce=(world > 1 and not args.nccl_allreduce))
    torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ops = ("dsmultT", "dsmult", "dds", "allreduce_exposed")
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            st.run()
        barrier()
        L.bidmat_b200_timing_reset()
        L.bidmat_b200_timing_enable(0 if args.no_kernel_timing else 1)
        sampler = ClockSampler(physical_index(local_rank))
        launches0 = L.bidmat_b200_launch_count()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(args.steps)]
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
            st.dsmult(); ev[s][2].record(stream)
            st.dds(); ev[s][3].record(stream)
            if work is not None:
                work.wait()
            ev[s][4].record(stream)
        t_end.record(stream)
        barrier()
        clocks = sampler.stop()
        launches = L.bidmat_b200_launch_count() - launches0
        L.bidmat_b200_timing_enable(0)
    total_ms = t_start.elapsed_time(t_end)
    op_ms = {o: sum(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(args.steps)) / args.steps
             for i, o in enumerate(ops)}
    kern = {}
    for label in ("dsmult_ga_chunk", "dsmultT_ga_chunk", "dsmultT_rowsort", "ga_fixup", "dds_chunk",
                  "sort_hist", "sort_scan", "sort_scatter"):
        ms, cnt = _lib.timing_read(label)
        kern[label] = {"launches_per_step": cnt / args.steps, "avg_ms": ms / cnt if cnt else None,
                       "ms_per_step": ms / args.steps}
    L.bidmat_b200_timing_reset()

    # max over ranks
    red = torch.tensor([total_ms] + [op_ms[o] for o in ops], dtype=torch.float64, device=dev)
    nnz_all = torch.tensor([shard.nnz], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(red, op=dist.ReduceOp.MAX)
        dist.all_reduce(nnz_all, op=dist.ReduceOp.SUM)
    total_ms = float(red[0])
    op_ms_max = {o: float(red[1 + i]) for i, o in enumerate(ops)}
    nnz_total = int(nnz_all[0])
    ms_per_step = total_ms / args.steps
    value = 3 * 2.0 * k * nnz_total / (ms_per_step * 1e-3) / 1e9

    # ----- end to end through the operator interface with host buffers (rank-local shard)
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, problem, shard, B_local, dev, world, group, GMat, GSMat, SMat, DDS)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    roof_ops = {}
    for o, label in (("dsmult", "dsmult_ga_chunk"), ("dds", "dds_chunk"), ("dsmultT", "dsmultT_ga_chunk")):
        # algorithmic bytes of the rank's whole shard; the launches of one step together process it once
        ab = algorithmic_bytes(o, k, shard.nnz, shard.n, m)
        ms = kern[label]["ms_per_step"]
        if o == "dsmultT" and world > 1:
            op_ms_max[o] += op_ms_max["allreduce_exposed"]   # the part of the allreduce that A*S and DDS did not hide
        roof_ops[o] = {"kernel": label, "kernel_ms": ms, "launches_per_step": kern[label]["launches_per_step"],
                       "algorithmic_bytes": ab,
                       "achieved_gbs": ab / (ms * 1e-3) / 1e9 if ms else None,
                       "frac": ab / (ms * 1e-3) / 1e9 / peak if ms else None,
                       "op_ms_max_over_ranks": op_ms_max[o],
                       "op_frac": ab / (op_ms_max[o] * 1e-3) / 1e9 / peak,
                       "op_gflops": 2.0 * k * nnz_total / (op_ms_max[o] * 1e-3) / 1e9}
    dom = max(roof_ops, key=lambda o: roof_ops[o]["kernel_ms"] or 0.0)
    roofline = {"bound": "hbm", "kernel": roof_ops[dom]["kernel"], "op": dom,
                "achieved": roof_ops[dom]["achieved_gbs"], "peak": peak, "unit": "GB/s",
                "frac": roof_ops[dom]["frac"], "peak_source": peak_src,
                "traffic": (MEASURED_DRAM_TRAFFIC[dom] if (world == 1 and args.scale == 1.0 and args.seed == 0
                                                          and not args.emulate_shard) else None),
                "traffic_note": "DRAM bytes per step of this operation's gather kernels, one-pass ncu capture of "
                                "this workload (summary committed under profiles/)",
                "ops": roof_ops, "kernels": kern}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": workload_config(problem, args, world),
        "clocks": clocks, "gpu_launches": int(launches), "roofline": roofline, "e2e": e2e,
        "allreduce_exposed_ms": op_ms_max["allreduce_exposed"] if world > 1 else 0.0,
        "allreduce": (None if world == 1 else
                      "library kernel over NVLink peer memory" if st.peer is not None else "NCCL"),
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args, problem)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_e2e(args, problem, shard, B_local, dev, world, group, GMat, GSMat, SMat, DDS):
    """Same three operations through the GMat/GSMat operator interface with
    HOST operands: every step uploads A, B and S from pinned memory, runs
    A*S, DDS and B*^S (+ allreduce) and downloads the three results.

    On several GPUs the replicated model A crosses PCIe once (rank 0 uploads it and
    broadcasts it over NVLink) and the reduced G, identical on every rank, is read
    back once (by rank 0); S, B, C and P are sharded, each rank moves its own part."""
    import torch.distributed as dist
    k = problem.k
    rank = dist.get_rank() if world > 1 else 0
    pin = lambda t: t.cpu().pin_memory()
    hA = pin(problem.A) if rank == 0 else None
    hB = pin(B_local)
    hjc, hir, hdata = pin(shard.jc), pin(shard.ir), pin(shard.data)
    hC = torch.empty((shard.n, k), dtype=torch.float32).pin_memory()
    hP = torch.empty(shard.nnz, dtype=torch.float32).pin_memory()
    hG = torch.empty((shard.m, k), dtype=torch.float32).pin_memory() if rank == 0 else None
    h2d = sum(t.numel() * t.element_size() for t in (hA, hB, hjc, hir, hdata) if t is not None)
    d2h = sum(t.numel() * t.element_size() for t in (hC, hP, hG) if t is not None)

    up = torch.cuda.Stream(device=dev)      # host -> device copies
    down = torch.cuda.Stream(device=dev)    # device -> host copies
    main = torch.cuda.current_stream(dev)

    def one():
        # Uploads are queued on their own stream in the order the operations need
        # them (S and A for A*S first, B last); each result starts its way back to
        # the host as soon as the operation that produced it has returned, so PCIe
        # runs in both directions while the next operation computes.
        with torch.cuda.stream(up):
            d_jc, d_ir, d_data = (h.to(dev, non_blocking=True) for h in (hjc, hir, hdata))
            if hA is not None:
                d_A = hA.to(dev, non_blocking=True)
            else:
                d_A = torch.empty((problem.m, k), dtype=torch.float32, device=dev)
            ev_sa = torch.cuda.Event(); ev_sa.record(up)
            d_B = hB.to(dev, non_blocking=True)
            ev_b = torch.cuda.Event(); ev_b.record(up)
        main.wait_event(ev_sa)
        if group is not None:
            dist.broadcast(d_A, src=0, group=group)     # the model reaches the other GPUs over NVLink
        A = GMat(d_A)
        S = GSMat.from_csc(shard.m, shard.n, d_jc, d_ir, d_data)
        C = A * S                                   # synchronous, like the BIDMat call
        with torch.cuda.stream(down):
            hC.copy_(C.t, non_blocking=True)
        main.wait_event(ev_b)
        B = GMat(d_B)
        G = B.xT(S)
        if group is not None:
            dist.all_reduce(G.t, op=dist.ReduceOp.SUM, group=group)
            torch.cuda.current_stream(dev).synchronize()
        if hG is not None:
            with torch.cuda.stream(down):
                hG.copy_(G.t, non_blocking=True)
        P = DDS(A, B, S)
        with torch.cuda.stream(down):
            hP.copy_(P.pdata, non_blocking=True)
        torch.cuda.synchronize()

    one()  # warm-up (allocator, workspace)
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
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(nnz, op=dist.ReduceOp.SUM)
        dist.all_reduce(bytes_, op=dist.ReduceOp.SUM)
    return {"value": 3 * 2.0 * k * float(nnz[0]) / (float(ms[0]) * 1e-3) / 1e9, "unit": UNIT,
            "ms_per_step": float(ms[0]), "steps": args.e2e_steps,
            "h2d_bytes_per_step": int(bytes_[0]), "d2h_bytes_per_step": int(bytes_[1]),
            "api": "GMat * GSMat, GMat.xT(GSMat), DDS(GMat, GMat, GSMat) with pinned host operands; "
                   "uploads and downloads on their own streams"}


def cpu_baseline(args, problem):
    threads = os.cpu_count() or 1
    sample, nnz, ncols = calibrated_sample(problem, args.cpu_seconds, threads)
    r = cpu_sample_run(sample, threads)
    k = problem.k
    total = sum(r.values())
    out = {"value": 3 * 2.0 * k * nnz / total / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
           "sample": "first %d columns (%d nonzeros) of the workload, each loop once; B*^S threaded over k-ranges "
                     "as FMat.maddT does (min(cores, k/32) threads)" % (ncols, nnz),
           "cpu_model": cpu_model(), "seconds": total,
           "ops_gflops": {o: 2.0 * k * nnz / r[o] / 1e9 for o in r}}
    try:
        import oracle
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
