"""Per-operation timing of the sparse-dense path on the benchmark
configurations other than the one bench.py reports (which is the LDA-shaped
configuration 2/4).  One JSON line per operation:

    python -m bidmat_b200.report --config 1
    python -m bidmat_b200.report --config 3 --k 32 64 128 256 512
    python -m bidmat_b200.report --config 5            (one GPU: the whole matrix)
    torchrun --nproc-per-node 8 -m bidmat_b200.report --config 5   (column shards + allreduce)

Times are CUDA events on the launching stream around the stream-ordered C ABI
calls, median of --reps after --warmup; inputs are resident on the device and
larger than L2 except where the configuration itself is small (config 1).
Flops follow BIDMat's convention 2*k*nnz per operation; the roofline fraction
is algorithmic bytes / time / measured HBM copy bandwidth.
"""
import argparse
import json
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def _alg_bytes(op, k, nnz, n, m):
    if op == "A*S":
        return nnz * (4 * k + 12) + n * 8 * k
    if op == "DDS":
        return nnz * (4 * k + 16) + n * 4 * k
    return nnz * (4 * k + 12) + m * 8 * k


def _time(fn, stream, reps, warmup):
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=2, choices=[1, 2, 3, 5])
    ap.add_argument("--extras", action="store_true",
                    help="time the operations around the path (transpose, sums, edge operators, tiles, fp64 twins) "
                         "on the LDA-shaped configuration at --scale (one GPU)")
    ap.add_argument("--k", type=int, nargs="*", default=[32, 64, 128, 256, 512])
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD

    from . import gen, step as pstep
    peak, peak_src = _peak()
    stream = torch.cuda.Stream(device=dev)
    if args.extras:
        return extras(args, dev, stream, peak, peak_src)

    if args.config == 3:
        problems = [(lambda kk=kk: gen.config3(kk, args.scale, args.seed, dev)) for kk in args.k]
    elif args.config == 1:
        problems = [lambda: gen.config1(args.scale, args.seed, dev)]
    elif args.config == 2:
        problems = [lambda: gen.config2(args.scale, args.seed, dev)]
    else:
        problems = [lambda: gen.config5(args.scale, args.seed, dev)]

    for make in problems:
        p = make()
        shard, _ = pstep.make_shard(p, rank, world)
        B_local = p.B[shard.col0:shard.col1].contiguous()
        st = pstep.PathStep(p.k, shard, p.A, B_local, stream, group)
        with torch.cuda.stream(stream):
            ops = []
            if args.config == 3:
                ops = [("DDS", st.dds)]
            elif args.config == 5:
                # P = DDS(A,B,S); C = A*S; G = B *^ P (P's values on S's pattern); allreduce G
                def g_of_p():
                    st.dsmultT(data=st.P)     # P has S's pattern: the plan of S serves it
                ops = [("DDS", st.dds), ("A*S", st.dsmult), ("B*^P", g_of_p)]
            else:
                ops = [("A*S", st.dsmult), ("DDS", st.dds), ("B*^S", st.dsmultT)]
            for name, fn in ops:
                ms = _time(fn, stream, args.reps, args.warmup)
                t = torch.tensor([ms], dtype=torch.float64, device=dev)
                nnz = torch.tensor([float(shard.nnz)], dtype=torch.float64, device=dev)
                if world > 1:
                    import torch.distributed as dist
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    dist.all_reduce(nnz, op=dist.ReduceOp.SUM)
                ms, nnz_total = float(t[0]), int(nnz[0])
                if rank == 0:
                    ab = _alg_bytes(name, p.k, shard.nnz, shard.n, p.m)
                    print(json.dumps({
                        "config": p.name, "op": name, "k": p.k, "m": p.m, "n": p.n, "nnz": nnz_total, "n_gpus": world,
                        "ms": ms, "gflops": 2.0 * p.k * nnz_total / (ms * 1e-3) / 1e9,
                        "nnz_k_per_s": p.k * nnz_total / (ms * 1e-3),
                        "roofline_frac": ab / (ms * 1e-3) / 1e9 / peak, "peak_gbs": peak, "peak_source": peak_src,
                        "scale": args.scale, "seed": args.seed}), flush=True)
        del st, shard, B_local, p
        torch.cuda.empty_cache()
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def extras(args, dev, stream, peak, peak_src):
    """Operations either side of the path, on device-resident operands, through the
    synchronous C ABI (each call ends with a stream synchronisation, as in BIDMat)."""
    from . import _lib, gen
    from .mat import GMat, GSMat
    L = _lib.lib
    p = gen.config2(args.scale, args.seed, dev)
    S = GSMat.from_csc(p.m, p.n, p.jc, p.ir, p.data)
    k, nnz, m, n = p.k, p.nnz, p.m, p.n
    A, B = GMat(p.A), GMat(p.B)
    rowv = torch.rand(n, device=dev) + 0.5
    colv = torch.rand(m, device=dev) + 0.5
    vals = p.data.clone()
    sums_c = torch.zeros(n, device=dev)
    sums_r = torch.zeros(m, device=dev)
    A64, B64 = p.A.double(), p.B.double()
    d64 = p.data.double()
    C64 = torch.zeros((n, k), dtype=torch.float64, device=dev)
    G64 = torch.zeros((m, k), dtype=torch.float64, device=dev)
    P64 = torch.zeros(nnz, dtype=torch.float64, device=dev)
    Ct = torch.zeros((n, k), device=dev)
    half_r, half_c = m // 2, n // 2
    ptr = lambda t: t.data_ptr()

    def ck(e):
        if e != 0:
            raise RuntimeError(_lib.error_string(e))

    import ctypes
    plan64 = ctypes.c_void_p(0)
    ck(L.bidmat_b200_dsmultT_plan_create(k, n, nnz, m, ptr(S.pir), ptr(S.pic), 8, None, ctypes.byref(plan64)))
    cases = [
        ("transpose (GSMat.t)", lambda: S.t, nnz * 24.0, None),
        ("spsum columns", lambda: ck(L.bidmat_b200_spsum(m, n, nnz, ptr(S.pir), ptr(S.pic), ptr(S.pdata), ptr(sums_c), 1)),
         nnz * 8.0 + n * 8.0, None),
        ("spsum rows", lambda: ck(L.bidmat_b200_spsum(m, n, nnz, ptr(S.pir), ptr(S.pic), ptr(S.pdata), ptr(sums_r), 2)),
         nnz * 8.0 + m * 8.0, None),
        ("sdoprow (*@ row vector)", lambda: ck(L.bidmat_b200_sdoprow(m, n, nnz, ptr(vals), ptr(S.pic), ptr(rowv), n, 2)),
         nnz * 12.0, None),
        ("sdopcol (*@ column vector)", lambda: ck(L.bidmat_b200_sdopcol(m, n, nnz, ptr(vals), ptr(S.pir), ptr(colv), m, 2)),
         nnz * 16.0, None),
        ("dsmultTile (whole matrix as one tile)",
         lambda: ck(L.bidmat_b200_dsmultTile(k, n, m, nnz, A.pdata, k, ptr(S.pdata), ptr(S.pir), ptr(S.pic), 0, 0, ptr(Ct), k, 0)),
         _alg_bytes("A*S", k, nnz, n, m), 2.0 * k * nnz),
        ("dsmultTile (lower-right quarter)",
         lambda: ck(L.bidmat_b200_dsmultTile(k, n - half_c, m - half_r, nnz, A.pdata + 4 * k * half_r, k, ptr(S.pdata),
                                             ptr(S.pir), ptr(S.pic), half_r, half_c, ptr(Ct) + 4 * k * half_c, k, 0)),
         None, None),
        ("A*S fp64", lambda: ck(L.bidmat_b200_dsmult_f64(k, n, nnz, ptr(A64), ptr(d64), ptr(S.pir), ptr(S.pic), ptr(C64))),
         nnz * (8.0 * k + 16) + n * 16.0 * k, 2.0 * k * nnz),
        ("DDS fp64", lambda: ck(L.bidmat_b200_dds_f64(k, nnz, ptr(A64), ptr(B64), ptr(S.pir), ptr(S.pic), ptr(P64))),
         nnz * (8.0 * k + 24) + n * 8.0 * k, 2.0 * k * nnz),
        ("B*^S fp64", lambda: ck(L.bidmat_b200_dsmultT_f64(k, n, nnz, ptr(B64), ptr(d64), ptr(S.pir), ptr(S.pic), ptr(G64))),
         nnz * (8.0 * k + 16) + m * 16.0 * k, 2.0 * k * nnz),
        ("B*^S fp64 (prepared plan)",
         lambda: (ck(L.bidmat_b200_dsmultT_planned_f64(plan64, k, n, nnz, ptr(B64), ptr(d64), ptr(G64), 0, None)),
                  torch.cuda.synchronize(dev)),
         nnz * (8.0 * k + 16) + m * 16.0 * k, 2.0 * k * nnz),
    ]
    for name, fn, nbytes, flops in cases:
        ms = _time(fn, torch.cuda.current_stream(dev), args.reps, args.warmup)
        out = {"config": p.name, "op": name, "k": k, "m": m, "n": n, "nnz": nnz, "n_gpus": 1, "ms": ms,
               "scale": args.scale, "seed": args.seed}
        if nbytes:
            out["algorithmic_gb"] = nbytes / 1e9
            out["roofline_frac"] = nbytes / (ms * 1e-3) / 1e9 / peak
            out["peak_gbs"], out["peak_source"] = peak, peak_src
        if flops:
            out["gflops"] = flops / (ms * 1e-3) / 1e9
        print(json.dumps(out), flush=True)
    ck(L.bidmat_b200_plan_destroy(plan64))
    return 0


if __name__ == "__main__":
    sys.exit(main())
