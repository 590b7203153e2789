// Kernels of the sparse-dense path: gather-accumulate over nonzero chunks (A*S
// and, on the row-sorted structure, B*^S), its deterministic fix-up, and the
// sampled dense-dense product.  sm_100a only; fp32 CUDA cores, no tensor cores:
// the work is a gather with 0.5 flop per byte.
#pragma once
#include "common.cuh"

namespace bidmat {

// ---------------------------------------------------------------------------
// Gather-accumulate:  O[:, seg[j]] += val[j] * D[:, gidx[j]]   for j in [0,nnz)
//
// `seg` is non-decreasing, so the nonzeros of one output column form one
// contiguous run.  The nonzero array is cut into chunks of `chunk` entries and
// each worker (LPV lanes) takes one chunk, which balances load by nonzeros
// whatever the column lengths are.  A run that lies inside one chunk is summed
// in registers and added to O by its only owner (plain load/add/store).  A run
// that crosses a chunk boundary is never added to O here: each chunk stores its
// piece of it in `part` (slot 0 of the chunk = piece of the run entering from
// the left, slot 1 = piece of the run leaving to the right) and ga_fixup_kernel
// adds the pieces in chunk order.  No float atomics anywhere, so the result is
// bit-reproducible.
//
// Dense column layout per worker: lane l holds VEC-wide elements l + t*LPV,
// t < NT, of the k-tile selected by blockIdx.y (tile width LPV*NT*VEC floats).
// ---------------------------------------------------------------------------
template <int VEC, int LPV, int NT, int U>
__global__ void __launch_bounds__(kThreads)
ga_chunk_kernel(int k, long long nnz, int chunk, long long nchunks,
                const float *__restrict__ D, const float *__restrict__ val,
                const int *__restrict__ gidx, const int *__restrict__ seg,
                float *__restrict__ O, float *__restrict__ part) {
    typedef Vec<VEC> V;
    typedef typename V::T VT;
    const int lane = threadIdx.x & (LPV - 1);
    const unsigned mask = worker_mask<LPV>();
    const long long c = ((long long)blockIdx.x * kThreads + threadIdx.x) / LPV;
    if (c >= nchunks) return;

    const int ktile = blockIdx.y * (LPV * NT * VEC);
    int eoff[NT];      // float offset of this lane's t-th element inside a column
    bool eok[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) {
        eoff[t] = ktile + (lane + t * LPV) * VEC;
        eok[t] = eoff[t] < k;
    }

    const long long j0 = c * (long long)chunk;
    const long long j1 = (j0 + chunk < nnz) ? j0 + chunk : nnz;
    int cur = __ldg(seg + j0);
    bool head_open = (j0 > 0) && (__ldg(seg + j0 - 1) == cur);

    VT acc[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t] = V::zero();

    auto flush = [&](bool tail_open) {
        if (!head_open && !tail_open) {
            float *o = O + (size_t)cur * k;
#pragma unroll
            for (int t = 0; t < NT; t++)
                if (eok[t]) {
                    VT old = V::ld(o + eoff[t]);
                    V::add(old, acc[t]);
                    V::st(o + eoff[t], old);
                }
        } else {
            float *p = part + ((size_t)c * 2 + (head_open ? 0 : 1)) * k;
#pragma unroll
            for (int t = 0; t < NT; t++)
                if (eok[t]) V::st(p + eoff[t], acc[t]);
        }
    };

    for (long long base = j0; base < j1; base += LPV) {
        long long jj = base + lane;
        if (jj >= j1) jj = j1 - 1;  // padded lanes repeat the last entry; never accumulated
        const int my_idx = __ldg(gidx + jj);
        const float my_val = __ldg(val + jj);
        const int my_seg = __ldg(seg + jj);
        const int cnt = (j1 - base < LPV) ? (int)(j1 - base) : LPV;
        for (int t0 = 0; t0 < cnt; t0 += U) {
            VT x[U][NT];
            int s[U];
            float v[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int src = (t0 + u) & (LPV - 1);
                const int i = __shfl_sync(mask, my_idx, src, LPV);
                v[u] = __shfl_sync(mask, my_val, src, LPV);
                s[u] = __shfl_sync(mask, my_seg, src, LPV);
                const float *d = D + (size_t)i * k;
#pragma unroll
                for (int t = 0; t < NT; t++) x[u][t] = eok[t] ? V::ldg(d + eoff[t]) : V::zero();
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                if (t0 + u < cnt) {
                    if (s[u] != cur) {
                        flush(false);
                        cur = s[u];
                        head_open = false;
#pragma unroll
                        for (int t = 0; t < NT; t++) acc[t] = V::zero();
                    }
#pragma unroll
                    for (int t = 0; t < NT; t++) V::fma(acc[t], v[u], x[u][t]);
                }
            }
        }
    }
    const bool tail_open = (j1 < nnz) && (__ldg(seg + j1) == cur);
    flush(tail_open);
}

// One worker per chunk.  The worker whose chunk holds the START of a run that
// leaves the chunk to the right walks the following chunks, adds the stored
// pieces in chunk order and adds the total to O.  Every other worker returns.
template <int VEC, int LPV, int NT>
__global__ void __launch_bounds__(kThreads)
ga_fixup_kernel(int k, long long nnz, int chunk, long long nchunks,
                const int *__restrict__ seg, float *__restrict__ O,
                const float *__restrict__ part) {
    typedef Vec<VEC> V;
    typedef typename V::T VT;
    const int lane = threadIdx.x & (LPV - 1);
    const long long c = ((long long)blockIdx.x * kThreads + threadIdx.x) / LPV;
    if (c >= nchunks) return;
    const long long j0 = c * (long long)chunk;
    const long long j1 = j0 + chunk;
    if (j1 >= nnz) return;
    const int s = __ldg(seg + j1 - 1);
    if (__ldg(seg + j1) != s) return;                       // nothing leaves to the right
    if (j0 > 0 && __ldg(seg + j0 - 1) == s) return;         // the run started further left

    const int ktile = blockIdx.y * (LPV * NT * VEC);
    int eoff[NT];
    bool eok[NT];
    VT tot[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) {
        eoff[t] = ktile + (lane + t * LPV) * VEC;
        eok[t] = eoff[t] < k;
        tot[t] = eok[t] ? V::ld(part + ((size_t)c * 2 + 1) * k + eoff[t]) : V::zero();
    }
    for (long long d = c + 1; d < nchunks; d++) {
        const float *p = part + (size_t)d * 2 * k;
#pragma unroll
        for (int t = 0; t < NT; t++)
            if (eok[t]) V::add(tot[t], V::ld(p + eoff[t]));
        const long long dj1 = (d + 1) * (long long)chunk;
        if (dj1 >= nnz) break;
        if (__ldg(seg + dj1 - 1) != s || __ldg(seg + dj1) != s) break;  // run ends in chunk d
    }
    float *o = O + (size_t)s * k;
#pragma unroll
    for (int t = 0; t < NT; t++)
        if (eok[t]) {
            VT old = V::ld(o + eoff[t]);
            V::add(old, tot[t]);
            V::st(o + eoff[t], old);
        }
}

// ---------------------------------------------------------------------------
// Sampled dense-dense product:  P[j] (+)= <A[:, ir[j]], B[:, ic[j]]>
//
// One worker per chunk of nonzeros.  The B column is kept in registers while
// the column index stays the same (ic is non-decreasing, so it is re-read
// about once per column); A columns are gathered U at a time with 16-byte
// loads; the dot product is finished with xor-shuffles inside the worker; the
// LPV results of one batch are written back as one coalesced store.
// A k-tile wider than LPV*NT*VEC is handled by looping over tiles inside the
// worker so that P is written once.
// ---------------------------------------------------------------------------
template <int VEC, int LPV, int NT, int U, bool ACCUM>
__global__ void __launch_bounds__(kThreads)
dds_chunk_kernel(int k, long long nnz, int chunk, long long nchunks,
                 const float *__restrict__ A, const float *__restrict__ B,
                 const int *__restrict__ ir, const int *__restrict__ ic, float *__restrict__ P) {
    typedef Vec<VEC> V;
    typedef typename V::T VT;
    const int lane = threadIdx.x & (LPV - 1);
    const unsigned mask = worker_mask<LPV>();
    const long long c = ((long long)blockIdx.x * kThreads + threadIdx.x) / LPV;
    if (c >= nchunks) return;
    constexpr int TILE = LPV * NT * VEC;
    const int ntiles = (k + TILE - 1) / TILE;

    const long long j0 = c * (long long)chunk;
    const long long j1 = (j0 + chunk < nnz) ? j0 + chunk : nnz;

    int cur = -1;  // column whose B vector is held in b[]
    VT b[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) b[t] = V::zero();

    for (long long base = j0; base < j1; base += LPV) {
        long long jj = base + lane;
        const bool mine_ok = jj < j1;
        if (!mine_ok) jj = j1 - 1;
        const int my_ir = __ldg(ir + jj);
        const int my_ic = __ldg(ic + jj);
        const int cnt = (j1 - base < LPV) ? (int)(j1 - base) : LPV;
        float mine = 0.f;
        for (int tile = 0; tile < ntiles; tile++) {
            int eoff[NT];
            bool eok[NT];
#pragma unroll
            for (int t = 0; t < NT; t++) {
                eoff[t] = tile * TILE + (lane + t * LPV) * VEC;
                eok[t] = eoff[t] < k;
            }
            if (ntiles > 1) cur = -1;  // b[] belongs to another tile
            for (int t0 = 0; t0 < cnt; t0 += U) {
                VT x[U][NT];
                int cc[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int src = (t0 + u) & (LPV - 1);
                    const int i = __shfl_sync(mask, my_ir, src, LPV);
                    cc[u] = __shfl_sync(mask, my_ic, src, LPV);
                    const float *a = A + (size_t)i * k;
#pragma unroll
                    for (int t = 0; t < NT; t++) x[u][t] = eok[t] ? V::ldg(a + eoff[t]) : V::zero();
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
                    if (t0 + u < cnt) {
                        if (cc[u] != cur) {
                            cur = cc[u];
                            const float *bp = B + (size_t)cur * k;
#pragma unroll
                            for (int t = 0; t < NT; t++) b[t] = eok[t] ? V::ldg(bp + eoff[t]) : V::zero();
                        }
                        float p = 0.f;
#pragma unroll
                        for (int t = 0; t < NT; t++) p = V::dot(x[u][t], b[t], p);
#pragma unroll
                        for (int off = LPV / 2; off > 0; off >>= 1) p += __shfl_xor_sync(mask, p, off, LPV);
                        if (lane == t0 + u) mine += p;
                    }
                }
            }
        }
        if (mine_ok) {
            if (ACCUM) P[jj] = P[jj] + mine;
            else P[jj] = mine;
        }
    }
}

}  // namespace bidmat
