// Stable LSD radix sort of the nonzero list by (column block, row), carrying
// (column, value) as payload: the CSC -> row-major reordering that makes the
// transposed product B*^S an atomic-free gather.
//
// key(j) = ((ic[j] >> colshift) << rowbits) | ir[j]      (unsigned 32 bit)
//
// One pass over an 8-bit digit is three kernels:
//   sort_hist_kernel     per-tile digit counts            counts[d][tile]
//   sort_scan_kernel     exclusive scan over (d, tile)    in place, two levels
//   sort_scatter_kernel  ranks every key of the tile among the tile's keys of
//                        the same digit in input order (warp match + per-warp
//                        counters), stages the tile digit-sorted in shared
//                        memory and writes runs of equal digits to consecutive
//                        addresses.
// Equal keys keep their input order in every pass, so within an output row the
// nonzeros stay in ascending source column: the order in which the reference
// CPU loop adds them.
#pragma once
#include "common.cuh"

namespace bidmat {

constexpr int kSortThreads = 256;                 // 8 warps
constexpr int kSortKeysPerThread = 16;
constexpr int kSortTile = kSortThreads * kSortKeysPerThread;   // 4096 keys per CTA
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortKeysPerWarp = kSortTile / kSortWarps;       // 512

struct SortKeySpec {
    int colshift;   // column block = ic >> colshift
    int rowbits;    // bits reserved for the row index
};

__device__ __forceinline__ unsigned make_sort_key(int row, int col, SortKeySpec ks) {
    return (((unsigned)col >> ks.colshift) << ks.rowbits) | (unsigned)row;
}

// FIRST: keys are computed from (ir, ic); otherwise read from keys_in.  In the first
// scatter pass a null value array makes the position of each nonzero its payload,
// which gives the permutation the sort applies.  A null column array (in and out)
// sorts (row, value) pairs only: 16 instead of 24 bytes per key and pass.
template <bool FIRST>
__global__ void __launch_bounds__(kSortThreads)
sort_hist_kernel(long long n, int ntiles, int shift, SortKeySpec ks, const unsigned *__restrict__ keys_in,
                 const int *__restrict__ ir, const int *__restrict__ ic, int *__restrict__ counts) {
    __shared__ int h[256];
    h[threadIdx.x] = 0;
    __syncthreads();
    const long long base = (long long)blockIdx.x * kSortTile;
    // Each thread folds runs of equal digits among its own keys before touching
    // shared memory, which removes most of the contention when one digit
    // dominates (integer counts: the order of the additions does not matter).
    unsigned prev = 0xffffffffu;
    int run = 0;
#pragma unroll 4
    for (int i = 0; i < kSortKeysPerThread; i++) {
        const long long j = base + i * kSortThreads + threadIdx.x;
        if (j < n) {
            const unsigned key = FIRST ? make_sort_key(__ldg(ir + j), ic ? __ldg(ic + j) : 0, ks) : __ldg(keys_in + j);
            const unsigned d = (key >> shift) & 255u;
            if (d == prev) {
                run++;
            } else {
                if (run) atomicAdd(&h[prev], run);
                prev = d;
                run = 1;
            }
        }
    }
    if (run) atomicAdd(&h[prev], run);
    __syncthreads();
    counts[(size_t)threadIdx.x * ntiles + blockIdx.x] = h[threadIdx.x];
}

// Exclusive scan over counts[d][tile] in (digit, tile) order, in two levels.
// Level 1: CTA (seg, d) scans tiles [seg*tps, (seg+1)*tps) of digit d in place
// and writes the segment total to seg_tot[d][seg].
constexpr int kSortScanSegs = 32;

static __global__ void __launch_bounds__(kSortThreads)
sort_scan_kernel(int ntiles, int tps, int *__restrict__ counts, int *__restrict__ seg_tot) {
    __shared__ int warp_sums[kSortWarps];
    __shared__ int carry_s;
    const int d = blockIdx.y, sg = blockIdx.x;
    const int t0 = sg * tps;
    const int t1 = (t0 + tps < ntiles) ? t0 + tps : ntiles;
    int *row = counts + (size_t)d * ntiles;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int base = t0; base < t1; base += kSortThreads) {
        const int i = base + threadIdx.x;
        const int v = (i < t1) ? row[i] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_sums[wid] = incl;
        __syncthreads();
        int woff = 0;
#pragma unroll
        for (int q = 0; q < kSortWarps; q++) woff += (q < wid) ? warp_sums[q] : 0;
        const int carry = carry_s;
        if (i < t1) row[i] = carry + woff + incl - v;
        __syncthreads();
        if (threadIdx.x == kSortThreads - 1) carry_s = carry + woff + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) seg_tot[d * kSortScanSegs + sg] = carry_s;
}

// Level 2 (one CTA, thread = digit): turns seg_tot[d][seg] into the output
// offset of the first key of digit d in segment seg.
static __global__ void __launch_bounds__(256) sort_digit_base_kernel(int *__restrict__ seg_tot) {
    __shared__ int s[256];
    const int d = threadIdx.x;
    int run = 0;
    for (int g = 0; g < kSortScanSegs; g++) {
        const int t = seg_tot[d * kSortScanSegs + g];
        seg_tot[d * kSortScanSegs + g] = run;
        run += t;
    }
    s[d] = run;
    __syncthreads();
    int base = 0;
    for (int i = 0; i < d; i++) base += s[i];
    for (int g = 0; g < kSortScanSegs; g++) seg_tot[d * kSortScanSegs + g] += base;
}

template <typename PV> struct SortSmem {
    PV b[kSortTile];                   // value payload (float or double), first for alignment
    unsigned key[kSortTile];
    int a[kSortTile];
    int warp_count[kSortWarps][256];   // per-warp digit counts, then exclusive offsets over warps
    int digit_start[256];              // first slot of each digit in the sorted tile
    int global_base[256];              // first output slot of this tile's keys of each digit
    int scan_tmp[kSortWarps];
};

template <bool FIRST, typename PV>
__global__ void __launch_bounds__(kSortThreads, (sizeof(PV) == 4 ? 3 : 2))
sort_scatter_kernel(long long n, int ntiles, int shift, SortKeySpec ks, const unsigned *__restrict__ keys_in,
                    const int *__restrict__ ir, const int *__restrict__ a_in, const PV *__restrict__ b_in,
                    const int *__restrict__ counts, const int *__restrict__ seg_base, int tps,
                    unsigned *__restrict__ keys_out, int *__restrict__ a_out, PV *__restrict__ b_out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SortSmem<PV> &sm = *reinterpret_cast<SortSmem<PV> *>(smem_raw);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long tile_base = (long long)blockIdx.x * kSortTile;
    const int tile_n = (int)((n - tile_base < kSortTile) ? (n - tile_base) : kSortTile);

    for (int i = threadIdx.x; i < kSortWarps * 256; i += kSortThreads) (&sm.warp_count[0][0])[i] = 0;
    sm.global_base[threadIdx.x] = seg_base[threadIdx.x * kSortScanSegs + blockIdx.x / tps] +
                                  counts[(size_t)threadIdx.x * ntiles + blockIdx.x];
    __syncthreads();

    // Warp `wid` owns tile positions [wid*512, wid*512+512); round r covers 32
    // consecutive positions, so (warp, round, lane) order is input order.
    unsigned key[kSortKeysPerThread];
    int pa[kSortKeysPerThread];
    PV pb[kSortKeysPerThread];
    int rank[kSortKeysPerThread];
#pragma unroll
    for (int r = 0; r < kSortKeysPerThread; r++) {
        const int pos = wid * kSortKeysPerWarp + r * 32 + lane;
        const bool ok = pos < tile_n;
        key[r] = 0;
        pa[r] = 0;
        pb[r] = 0;
        if (ok) {
            const long long j = tile_base + pos;
            pa[r] = a_in ? __ldg(a_in + j) : 0;          // no column payload: rows and values only
            pb[r] = b_in ? __ldg(b_in + j) : (PV)j;      // no payload given: the position itself
            key[r] = FIRST ? make_sort_key(__ldg(ir + j), pa[r], ks) : __ldg(keys_in + j);
        }
    }
#pragma unroll
    for (int r = 0; r < kSortKeysPerThread; r++) {
        const int pos = wid * kSortKeysPerWarp + r * 32 + lane;
        const bool ok = pos < tile_n;
        const unsigned valid = __ballot_sync(0xffffffffu, ok);
        rank[r] = 0;
        if (ok) {
            const unsigned d = (key[r] >> shift) & 255u;
            // lanes of this round holding the same digit: eight ballots, one per digit bit
            unsigned peers = valid;
#pragma unroll
            for (int bit = 0; bit < 8; bit++) {
                const bool one = (d >> bit) & 1u;
                const unsigned bal = __ballot_sync(valid, one);
                peers &= one ? bal : ~bal;
            }
            const int prior = sm.warp_count[wid][d];
            rank[r] = prior + __popc(peers & ((1u << lane) - 1u));
            __syncwarp(valid);
            if (lane == (__ffs(peers) - 1)) sm.warp_count[wid][d] = prior + __popc(peers);
        }
        __syncwarp(0xffffffffu);
    }
    __syncthreads();

    // digit = threadIdx.x: exclusive offsets over warps, tile total per digit
    int total = 0;
#pragma unroll
    for (int q = 0; q < kSortWarps; q++) {
        const int t = sm.warp_count[q][threadIdx.x];
        sm.warp_count[q][threadIdx.x] = total;
        total += t;
    }
    // exclusive scan of the 256 tile totals -> digit_start
    int incl = total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) sm.scan_tmp[wid] = incl;
    __syncthreads();
    int woff = 0;
#pragma unroll
    for (int q = 0; q < kSortWarps; q++) woff += (q < wid) ? sm.scan_tmp[q] : 0;
    sm.digit_start[threadIdx.x] = woff + incl - total;
    __syncthreads();

#pragma unroll
    for (int r = 0; r < kSortKeysPerThread; r++) {
        const int pos = wid * kSortKeysPerWarp + r * 32 + lane;
        if (pos < tile_n) {
            const unsigned d = (key[r] >> shift) & 255u;
            const int slot = sm.digit_start[d] + sm.warp_count[wid][d] + rank[r];
            sm.key[slot] = key[r];
            sm.a[slot] = pa[r];
            sm.b[slot] = pb[r];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < tile_n; i += kSortThreads) {
        const unsigned kk = sm.key[i];
        const unsigned d = (kk >> shift) & 255u;
        const long long out = (long long)sm.global_base[d] + (i - sm.digit_start[d]);
        keys_out[out] = kk;
        if (a_out) a_out[out] = sm.a[i];
        b_out[out] = sm.b[i];
    }
}

// largest row index: block reduction + integer atomicMax
static __global__ void __launch_bounds__(256) max_int_kernel(long long n, const int *__restrict__ v, int *__restrict__ out) {
    int m = -2147483647 - 1;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int x = __ldg(v + i);
        m = x > m ? x : m;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const int t = __shfl_xor_sync(0xffffffffu, m, o);
        m = t > m ? t : m;
    }
    if ((threadIdx.x & 31) == 0) atomicMax(out, m);
}

// off[b] = first sorted position whose key has column block >= b, b in [0, nblocks]
static __global__ void __launch_bounds__(256)
block_offsets_kernel(long long n, int nblocks, int rowbits, const unsigned *__restrict__ keys, int *__restrict__ off) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b > nblocks) return;
    const unsigned long long target = (unsigned long long)b << rowbits;
    long long lo = 0, hi = n;   // first position with key >= target
    while (lo < hi) {
        const long long mid = (lo + hi) >> 1;
        if ((unsigned long long)__ldg(keys + mid) < target) lo = mid + 1; else hi = mid;
    }
    off[b] = (int)lo;
}

}  // namespace bidmat
