// Kernels of the prepared ("planned") transposed product B*^S.
//
// A plan holds, for one sparse structure, the nonzero list sorted by
// (column block, row) with the source column and the original position of every
// nonzero, cut into chunks whose boundaries sit on row boundaries wherever a run
// of equal rows is shorter than a chunk.  A call then only has to bring the
// values into sorted order (one gather through the stored positions) and run the
// gather-accumulate kernel block after block: no sort, no host round trip.
// Runs longer than a chunk are split; their pieces go to numbered slots and one
// fix-up launch after the last block adds them, in chunk order, to the output.
#pragma once
#include "kernels.cuh"

namespace bidmat {

// ---------------------------------------------------------------------------
// Chunk boundaries.  The nonzeros [lo, hi) of one column block are sorted by key.
// Nominal boundaries sit at lo + c*T; boundary c is moved back to the start of
// the run of equal keys that contains it, unless that run began at or before the
// previous nominal boundary (then the run is longer than a chunk and is cut at
// the nominal position).  Every chunk is non-empty and shorter than 2T.
// Outputs, for c in [0, nch]: start[c], the key at start[c] (first[c]) and the key
// just before it (prev[c]); c = nch describes the end of the block.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
plan_bounds_kernel(int lo, int hi, int T, int nch, const unsigned *__restrict__ keys,
                   int *__restrict__ start, unsigned *__restrict__ first, unsigned *__restrict__ prev) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c > nch) return;
    int b;
    if (c == 0) b = lo;
    else if (c == nch) b = hi;
    else {
        const int p = lo + c * T;                 // < hi because nch = ceil((hi-lo)/T)
        const unsigned key = __ldg(keys + p);
        int a = lo, z = p;                        // first position in [lo, p] holding `key`
        while (a < z) {
            const int mid = (a + z) >> 1;
            if (__ldg(keys + mid) < key) a = mid + 1; else z = mid;
        }
        b = (a > lo + (c - 1) * T) ? a : p;
    }
    start[c] = b;
    first[c] = (b < hi) ? __ldg(keys + b) : 0xffffffffu;
    prev[c] = (b > lo) ? __ldg(keys + b - 1) : 0xffffffffu;
}

// vals[j] = data[perm[j]]: the values of a call, brought into the plan's order.
// mismatch (optional): set to 1 when the structure handed in with the call is not
// the one the plan was made for (row or column of a nonzero differs).
template <typename S>
__global__ void __launch_bounds__(256)
plan_permute_kernel(long long n, const int *__restrict__ perm, const S *__restrict__ data, S *__restrict__ vals) {
    // four independent position -> value chains per thread and iteration: the gathers are
    // 4- or 8-byte reads at scattered addresses, bound by the number of requests in flight
    constexpr int UN = 4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; j + (UN - 1) * stride < n; j += UN * stride) {
        int p[UN];
        S v[UN];
#pragma unroll
        for (int u = 0; u < UN; u++) p[u] = __ldg(perm + j + u * stride);
#pragma unroll
        for (int u = 0; u < UN; u++) v[u] = __ldg(data + p[u]);
#pragma unroll
        for (int u = 0; u < UN; u++) vals[j + u * stride] = v[u];
    }
    for (; j < n; j += stride) vals[j] = __ldg(data + __ldg(perm + j));
}

// The same permutation written as a scatter: vals[inv[i]] = data[i] with coalesced reads.
// Consecutive source positions are the nonzeros of one column in ascending row; the
// nonzeros of a frequent row in neighbouring columns land next to each other in the
// sorted list, so their 4-byte writes meet in the same L2 sectors shortly after one
// another, where the gather form misses on every access.
template <typename S>
__global__ void __launch_bounds__(256)
plan_scatter_kernel(long long n, const int *__restrict__ inv, const S *__restrict__ data, S *__restrict__ vals) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        vals[__ldg(inv + i)] = __ldg(data + i);
}

// inv[perm[j]] = j
__global__ void __launch_bounds__(256)
plan_invert_kernel(long long n, const int *__restrict__ perm, int *__restrict__ inv) {
    const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (j < n) inv[__ldg(perm + j)] = (int)j;
}

// Exact check that (ir, ic) is the structure a plan was built from: every sorted
// entry must name the row and column found at its stored source position.
__global__ void __launch_bounds__(256)
plan_verify_kernel(long long n, const int *__restrict__ perm, const unsigned *__restrict__ keys,
                   const int *__restrict__ cols, unsigned rowmask, const int *__restrict__ ir,
                   const int *__restrict__ ic, int *__restrict__ mismatch) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    bool bad = false;
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) {
        const int p = __ldg(perm + j);
        bad |= ((unsigned)__ldg(ir + p) != (__ldg(keys + j) & rowmask)) | (__ldg(ic + p) != __ldg(cols + j));
    }
    if (bad) *mismatch = 1;
}

// first_block[row] = lowest column block that holds a nonzero of the row (integer
// atomicMin at plan time only); rows nobody names keep kNoBlock (what a byte-wise
// memset with 0x7f leaves).
constexpr int kNoBlock = 0x7f7f7f7f;
__global__ void __launch_bounds__(256)
plan_first_block_kernel(long long n, const unsigned *__restrict__ keys, int rowbits, unsigned rowmask,
                        int *__restrict__ first_block, unsigned long long *__restrict__ nruns) {
    const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    // only the first nonzero of a run (one row inside one column block) needs to vote
    bool start = false;
    unsigned key = 0;
    if (j < n) {
        key = __ldg(keys + j);
        start = (j == 0) || (__ldg(keys + j - 1) != key);
    }
    if (start) atomicMin(first_block + (key & rowmask), (int)(key >> rowbits));
    const unsigned bal = __ballot_sync(0xffffffffu, start);
    if ((threadIdx.x & 31) == 0 && bal) atomicAdd(nruns, (unsigned long long)__popc(bal));   // number of runs
}

// Marks (bit 31 of the key) every nonzero that belongs to the first block of its
// row: in overwrite mode the run holding it stores instead of adding.  Rows whose
// first run is split over chunks (listed in `no_store`, 1 per row) are left
// unmarked: the call clears them and accumulates.
__global__ void __launch_bounds__(256)
plan_mark_first_kernel(long long n, unsigned *__restrict__ keys, int rowbits, unsigned rowmask,
                       const int *__restrict__ first_block, const unsigned char *__restrict__ no_store) {
    const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const unsigned key = keys[j];
    const unsigned row = key & rowmask;
    if ((int)(key >> rowbits) == first_block[row] && !no_store[row]) keys[j] = key | 0x80000000u;
}

// touched[w] bit b = row 32*w + b is named by at least one nonzero.
__global__ void __launch_bounds__(256)
plan_touched_kernel(int m, const int *__restrict__ first_block, unsigned *__restrict__ touched) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    const bool t = (row < m) && (first_block[row] != kNoBlock);
    const unsigned bal = __ballot_sync(0xffffffffu, t);
    if ((threadIdx.x & 31) == 0 && row < m) touched[row >> 5] = bal;
}

// Zeroes the output columns listed in rows[] (one worker of 32 lanes per column).
template <typename S>
__global__ void __launch_bounds__(256)
plan_clear_rows_kernel(int k, int nrows_listed, const int *__restrict__ rows, S *__restrict__ O) {
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (w >= nrows_listed) return;
    S *o = O + (size_t)__ldg(rows + w) * k;
    for (int i = threadIdx.x & 31; i < k; i += 32) o[i] = (S)0;
}

// Zeroes the output columns of the rows that no nonzero names (bitmap `touched`): one
// worker of 32 lanes per row.
template <typename S>
__global__ void __launch_bounds__(256)
plan_clear_untouched_kernel(int k, int m, const unsigned *__restrict__ touched, S *__restrict__ O) {
    const int row = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    if (row >= m) return;
    if ((__ldg(touched + (row >> 5)) >> (row & 31)) & 1u) return;
    S *o = O + (size_t)row * k;
    for (int i = threadIdx.x & 31; i < k; i += 32) o[i] = (S)0;
}

__device__ __forceinline__ void prefetch_l2(const void *p) {
    asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p));
}

// ---------------------------------------------------------------------------
// Gather-accumulate over the chunks of a plan, dense heights k = VEC*LPV*NT (fp32 or
// fp64, FUSED for fp32 only) with 16-byte aligned operands (the shapes of ga_chunk_fast_kernel, which this kernel
// follows: cp.async-staged (index, value, segment) triples, gathers U columns
// ahead of the FMAs, read half of the output's read-modify-write issued when a
// run starts).  Differences:
//   * chunk c of the launch is desc[c] = {first nonzero, end, slot of the piece
//     entering from the left or -1, slot of the piece leaving to the right / -1
//     nothing leaves / -2 the whole chunk is one run that goes on};
//   * the rows of the transposed product are short runs (often a single nonzero),
//     so the read of the output column would be a DRAM round trip per run on the
//     critical path: while batch b is processed, the output columns of the runs
//     that START in batch b+1 are prefetched into L2 (no registers held);
//   * a run whose segment value has `storebit` set overwrites its output column;
//   * FUSED: `val` is the caller's value array in its own (CSC) order and `perm` the
//     source position of every sorted nonzero.  The positions are staged two batches
//     ahead and the values one batch ahead through them, so the scattered 4-byte reads
//     (each a DRAM sector) overlap the gathers of this kernel, which leaves DRAM mostly
//     idle, instead of costing a pass of their own (plan_permute_kernel).
// ---------------------------------------------------------------------------
template <typename S, int LPV, int NT, int U, int TPB, int MINB, bool PREFETCH, bool FUSED>
__global__ void __launch_bounds__(TPB, MINB)
ga_plan_fast_kernel(int nchunks, const int4 *__restrict__ desc,
                    const S *__restrict__ D, const S *__restrict__ val, const int *__restrict__ perm,
                    const int *__restrict__ gidx, const int *__restrict__ seg,
                    S *__restrict__ O, S *__restrict__ part, unsigned segmask, unsigned storebit) {
    typedef FastOps<S> F;
    typedef typename F::vec vec;
    static_assert(!FUSED || sizeof(S) == 4, "the staged record has room for a position only beside a 4-byte value");
    constexpr int K = F::VEC * LPV * NT;
    constexpr int WPB = TPB / LPV;
    constexpr int G = LPV / U;
    constexpr int LINES = (K * (int)sizeof(S) + 127) / 128;     // 128-byte lines per output column
    constexpr int NBUF = FUSED ? 3 : 2;            // staged batches of {index, value, segment, position}
    static_assert(LPV % U == 0, "U must divide LPV");
    __shared__ int4 meta[WPB][NBUF][LPV];

    const int lane = threadIdx.x & (LPV - 1);
    const int w = threadIdx.x / LPV;
    const unsigned mask = worker_mask<LPV>();
    const int c = blockIdx.x * WPB + w;
    if (c >= nchunks) return;

    const int4 dc = __ldg(desc + c);
    const long long j0 = dc.x, j1 = dc.y;
    const int nb = (int)((j1 - j0 + LPV - 1) / LPV);
    const S *Dl = D + lane * F::VEC;

    // Every call commits exactly one cp.async group, also for a batch beyond the chunk
    // (an empty group), so the wait counts below do not depend on where the chunk ends.
    auto stage = [&](int batch) {                  // indices, segments and values or (FUSED) positions
        if (batch < nb) {
            const long long jj = j0 + (long long)batch * LPV + lane;
            int4 *dst = &meta[w][batch % NBUF][lane];
            if (jj < j1) {
                cp_async4(&dst->x, gidx + jj);
                F::stage_seg(dst, seg + jj);
                if (FUSED) cp_async4(&dst->w, perm + jj);
                else F::stage_val(dst, val + jj);
            } else {
                // padding of the last batch: repeat the last nonzero with value 0
                *dst = F::pad(__ldg(gidx + j1 - 1), __ldg(seg + j1 - 1));
            }
        }
        cp_async_commit();
    };
    auto stage_values = [&](int batch) {           // FUSED: values through the positions staged before
        if (batch < nb) {
            const long long jj = j0 + (long long)batch * LPV + lane;
            int4 *dst = &meta[w][batch % NBUF][lane];
            if (jj < j1) F::stage_val(dst, val + dst->w);      // this lane's own position: visible after its wait
        }
        cp_async_commit();
    };

    int cur = __ldg(seg + j0);
    bool head_open = dc.z >= 0;
    vec acc[NT];
    vec oldv[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) { acc[t] = F::zero(); oldv[t] = acc[t]; }

    auto prefetch_out = [&]() {
        if (((unsigned)cur & storebit) == 0u) {
            const vec *o = reinterpret_cast<const vec *>(O + (size_t)((unsigned)cur & segmask) * K) + lane;
#pragma unroll
            for (int t = 0; t < NT; t++) oldv[t] = o[t * LPV];
        }
    };

    auto flush = [&](bool tail_open) {
        if (!head_open && !tail_open) {
            vec *o = reinterpret_cast<vec *>(O + (size_t)((unsigned)cur & segmask) * K) + lane;
            if (((unsigned)cur & storebit) != 0u) {
#pragma unroll
                for (int t = 0; t < NT; t++) o[t * LPV] = acc[t];
            } else {
#pragma unroll
                for (int t = 0; t < NT; t++) {
                    vec old = oldv[t];
                    F::add(old, acc[t]);
                    o[t * LPV] = old;
                }
            }
        } else {
            vec *p = reinterpret_cast<vec *>(part + (size_t)(head_open ? dc.z : dc.w) * K) + lane;
#pragma unroll
            for (int t = 0; t < NT; t++) p[t * LPV] = acc[t];
        }
    };

    stage(0);
    if (FUSED) {
        stage(1);
        cp_async_wait<1>();        // positions of batch 0 are in
        stage_values(0);
    }
    if (PREFETCH) {
        // output columns of the runs that start in the first batch (the one entering
        // from the left, if any, goes to a slot and needs none)
        const bool v0 = j0 + lane < j1;
        const int s0 = v0 ? __ldg(seg + j0 + lane) : 0;
        int p0 = __shfl_up_sync(mask, s0, 1, LPV);
        if (lane == 0) p0 = head_open ? s0 : ~s0;
        if (v0 && s0 != p0 && ((unsigned)s0 & storebit) == 0u) {
            const char *o = reinterpret_cast<const char *>(O + (size_t)((unsigned)s0 & segmask) * K);
#pragma unroll
            for (int i = 0; i < LINES; i++) prefetch_l2(o + i * 128);
        }
    }
    if (!head_open) prefetch_out();
    for (int b = 0; b < nb; b++) {
        int nseg = 0;
        bool nvalid = false;
        if (PREFETCH && b + 1 < nb) {
            const long long nbase = j0 + (long long)(b + 1) * LPV;
            nvalid = nbase + lane < j1;
            nseg = nvalid ? __ldg(seg + nbase + lane) : 0;         // consumed half a batch later
        }
        if (FUSED) {
            // groups in commit order: ... P(b+1) V(b) | P(b+2) V(b+1)   (P positions+indices, V values)
            stage(b + 2);
            cp_async_wait<2>();        // all but V(b), P(b+2): the positions of batch b+1 are in
            stage_values(b + 1);
            cp_async_wait<2>();        // all but P(b+2), V(b+1): batch b is complete
        } else {
            stage(b + 1);
            cp_async_wait<1>();
        }
        worker_sync<LPV>(mask);
        const int4 *mt = meta[w][b % NBUF];

        vec x[2][U][NT];
        int4 e[2][U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            e[0][u] = mt[u];
            const vec *d = reinterpret_cast<const vec *>(Dl + (size_t)e[0][u].x * K);
#pragma unroll
            for (int t = 0; t < NT; t++) x[0][u][t] = __ldg(d + t * LPV);
        }
#pragma unroll
        for (int g = 0; g < G; g++) {
            if (g + 1 < G) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    e[(g + 1) & 1][u] = mt[(g + 1) * U + u];
                    const vec *d = reinterpret_cast<const vec *>(Dl + (size_t)e[(g + 1) & 1][u].x * K);
#pragma unroll
                    for (int t = 0; t < NT; t++) x[(g + 1) & 1][u][t] = __ldg(d + t * LPV);
                }
            }
            if (PREFETCH && g == G / 2) {
                // output columns of the runs that start in the next batch, into L2
                int pseg = __shfl_up_sync(mask, nseg, 1, LPV);
                if (lane == 0) pseg = F::seg(mt[LPV - 1]);
                if (nvalid && nseg != pseg && ((unsigned)nseg & storebit) == 0u) {
                    const char *o = reinterpret_cast<const char *>(O + (size_t)((unsigned)nseg & segmask) * K);
#pragma unroll
                    for (int i = 0; i < LINES; i++) prefetch_l2(o + i * 128);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int4 m = e[g & 1][u];
                if (F::seg(m) != cur) {
                    flush(false);
                    cur = F::seg(m);
                    head_open = false;
                    prefetch_out();
#pragma unroll
                    for (int t = 0; t < NT; t++) acc[t] = F::zero();
                }
                const S v = F::val(m);
#pragma unroll
                for (int t = 0; t < NT; t++) F::axpy(v, x[g & 1][u][t], acc[t]);
            }
        }
        worker_sync<LPV>(mask);
    }
    flush(dc.w != -1);
}

// ---------------------------------------------------------------------------
// Fix-up of a plan, in two launches and without float atomics.
//  1. plan_fixup_runs_kernel: one worker per split run {segment value, first slot,
//     number of pieces}.  The pieces lie in consecutive slots in chunk order; they are
//     added in that order and the total replaces the first piece.
//  2. plan_fixup_rows_kernel: one worker per output column that has split runs
//     {segment value, first run, number of runs}: a row of the sparse matrix can be
//     split in several column blocks, so its run totals are added here, by one worker,
//     in block order, and the sum is added to the output column once.  (Letting every
//     run update the output itself would race between the runs of one row.)
// ---------------------------------------------------------------------------
template <typename S, int VEC, int LPV, int NT>
__global__ void __launch_bounds__(kThreads)
plan_fixup_runs_kernel(int k, int nruns, const int4 *__restrict__ runs, S *__restrict__ part) {
    typedef Vec<S, VEC> V;
    typedef typename V::T VT;
    const int lane = threadIdx.x & (LPV - 1);
    const int r = (int)(((long long)blockIdx.x * kThreads + threadIdx.x) / LPV);
    if (r >= nruns) return;
    const int4 run = __ldg(runs + r);
    const int ktile = blockIdx.y * (LPV * NT * VEC);
    int eoff[NT];
    bool eok[NT];
    VT tot[NT];
    S *p = part + (size_t)run.y * k;
#pragma unroll
    for (int t = 0; t < NT; t++) {
        eoff[t] = ktile + (lane + t * LPV) * VEC;
        eok[t] = eoff[t] < k;
        tot[t] = eok[t] ? V::ld(p + eoff[t]) : V::zero();
    }
    constexpr int PF = 4;
    for (int q0 = 1; q0 < run.z; q0 += PF) {
        VT x[PF][NT];
#pragma unroll
        for (int q = 0; q < PF; q++) {
            const int qq = (q0 + q < run.z) ? q0 + q : run.z - 1;
            const S *pq = p + (size_t)qq * k;
#pragma unroll
            for (int t = 0; t < NT; t++) x[q][t] = eok[t] ? V::ld(pq + eoff[t]) : V::zero();
        }
#pragma unroll
        for (int q = 0; q < PF; q++)
            if (q0 + q < run.z) {
#pragma unroll
                for (int t = 0; t < NT; t++) V::add(tot[t], x[q][t]);
            }
    }
#pragma unroll
    for (int t = 0; t < NT; t++)
        if (eok[t]) V::st(p + eoff[t], tot[t]);
}

template <typename S, int VEC, int LPV, int NT>
__global__ void __launch_bounds__(kThreads)
plan_fixup_rows_kernel(int k, int ngroups, const int4 *__restrict__ groups, const int4 *__restrict__ runs,
                       S *__restrict__ O, const S *__restrict__ part, unsigned segmask) {
    typedef Vec<S, VEC> V;
    typedef typename V::T VT;
    const int lane = threadIdx.x & (LPV - 1);
    const int g = (int)(((long long)blockIdx.x * kThreads + threadIdx.x) / LPV);
    if (g >= ngroups) return;
    const int4 grp = __ldg(groups + g);
    const int ktile = blockIdx.y * (LPV * NT * VEC);
    int eoff[NT];
    bool eok[NT];
    VT tot[NT], old[NT];
    S *o = O + (size_t)((unsigned)grp.x & segmask) * k;
#pragma unroll
    for (int t = 0; t < NT; t++) {
        eoff[t] = ktile + (lane + t * LPV) * VEC;
        eok[t] = eoff[t] < k;
        old[t] = eok[t] ? V::ld(o + eoff[t]) : V::zero();
        tot[t] = V::zero();
    }
    for (int r = 0; r < grp.z; r++) {
        const S *p = part + (size_t)__ldg(&runs[grp.y + r].y) * k;
#pragma unroll
        for (int t = 0; t < NT; t++)
            if (eok[t]) { VT x = V::ld(p + eoff[t]); V::add(tot[t], x); }
    }
#pragma unroll
    for (int t = 0; t < NT; t++)
        if (eok[t]) {
            V::add(old[t], tot[t]);
            V::st(o + eoff[t], old[t]);
        }
}

}  // namespace bidmat
