// Stable compaction of the nonzeros of a GSMat that fall inside a tile
// [roff, roff+nrt) x [coff, coff+nct), with tile-relative indices, for the
// tiled products.  Included by one translation unit only.
#pragma once
#include "common.cuh"

namespace bidmat {

constexpr int kCompactThreads = 256;
constexpr int kCompactPerThread = 8;
constexpr int kCompactTile = kCompactThreads * kCompactPerThread;   // 2048 nonzeros per CTA

__device__ __forceinline__ bool in_tile(int r, int c, int roff, int nrt, int coff, int nct) {
    return (unsigned)(r - roff) < (unsigned)nrt && (unsigned)(c - coff) < (unsigned)nct;
}

// counts[t] = nonzeros of tile-of-the-list t that lie inside the matrix tile
__global__ void __launch_bounds__(kCompactThreads)
compact_count_kernel(long long nnz, const int *__restrict__ ir, const int *__restrict__ ic, int roff, int nrt,
                     int coff, int nct, int *__restrict__ counts) {
    __shared__ int total;
    if (threadIdx.x == 0) total = 0;
    __syncthreads();
    const long long base = (long long)blockIdx.x * kCompactTile;
    int mine = 0;
#pragma unroll
    for (int i = 0; i < kCompactPerThread; i++) {
        const long long j = base + i * kCompactThreads + threadIdx.x;
        if (j < nnz && in_tile(__ldg(ir + j), __ldg(ic + j), roff, nrt, coff, nct)) mine++;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if ((threadIdx.x & 31) == 0 && mine) atomicAdd(&total, mine);   // integer count
    __syncthreads();
    if (threadIdx.x == 0) counts[blockIdx.x] = total;
}

// In-place exclusive scan of counts[0..n) by one CTA; the grand total goes to counts[n].
__global__ void __launch_bounds__(1024) compact_scan_kernel(int n, int *__restrict__ counts) {
    __shared__ int warp_sums[32];
    __shared__ int carry_s;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int base = 0; base < n; base += 1024) {
        const int i = base + threadIdx.x;
        const int v = (i < n) ? counts[i] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_sums[wid] = incl;
        __syncthreads();
        int woff = 0;
        for (int q = 0; q < wid; q++) woff += warp_sums[q];
        const int carry = carry_s;
        if (i < n) counts[i] = carry + woff + incl - v;
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = carry + woff + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[n] = carry_s;
}

// Writes the in-tile nonzeros, in their original order, as (row - roff, col - coff, value).
// Positions inside a CTA follow (round, thread) order = list order.
template <typename S>
__global__ void __launch_bounds__(kCompactThreads)
compact_scatter_kernel(long long nnz, const int *__restrict__ ir, const int *__restrict__ ic,
                       const S *__restrict__ v, int roff, int nrt, int coff, int nct,
                       const int *__restrict__ offsets, int *__restrict__ orow, int *__restrict__ ocol,
                       S *__restrict__ oval) {
    __shared__ int warp_cnt[kCompactThreads / 32];
    __shared__ int running;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (threadIdx.x == 0) running = offsets[blockIdx.x];
    __syncthreads();
    const long long base = (long long)blockIdx.x * kCompactTile;
    for (int i = 0; i < kCompactPerThread; i++) {
        const long long j = base + i * kCompactThreads + threadIdx.x;
        int r = 0, c = 0;
        bool ok = false;
        if (j < nnz) {
            r = __ldg(ir + j);
            c = __ldg(ic + j);
            ok = in_tile(r, c, roff, nrt, coff, nct);
        }
        const unsigned bal = __ballot_sync(0xffffffffu, ok);
        if (lane == 0) warp_cnt[wid] = __popc(bal);
        __syncthreads();
        int woff = 0, round_total = 0;
#pragma unroll
        for (int q = 0; q < kCompactThreads / 32; q++) {
            const int cq = warp_cnt[q];
            woff += (q < wid) ? cq : 0;
            round_total += cq;
        }
        const int start = running;
        if (ok) {
            const int pos = start + woff + __popc(bal & ((1u << lane) - 1u));
            orow[pos] = r - roff;
            ocol[pos] = c - coff;
            oval[pos] = __ldg(v + j);
        }
        __syncthreads();
        if (threadIdx.x == 0) running = start + round_total;
        __syncthreads();
    }
}

}  // namespace bidmat
