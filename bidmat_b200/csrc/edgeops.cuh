// Edge operations on the values of a GSMat that sit either side of DDS in
// factorisation loops: value <- op(value, vector[row or column]), and the sums of
// the values over rows or columns.  Included by one translation unit only.
#pragma once
#include "common.cuh"

namespace bidmat {

// BIDMat's binary operator table (jni/src/Operators.cu:86-101), by index.
template <typename S> __device__ __forceinline__ S apply_binop(int opn, S a, S b) {
    switch (opn) {
        case 0: return a + b;
        case 1: return a - b;
        case 2: return a * b;
        case 3: return a / b;
        case 4: return (a > b) ? (S)1 : (S)0;
        case 5: return (a < b) ? (S)1 : (S)0;
        case 6: return (a == b) ? (S)1 : (S)0;
        case 7: return (a >= b) ? (S)1 : (S)0;
        case 8: return (a <= b) ? (S)1 : (S)0;
        case 9: return (a != b) ? (S)1 : (S)0;
        case 10: return fmax(a, b);
        case 11: return fmin(a, b);
        case 12: return atan2(a, b);
        case 13: return pow(a, b);
        default: return (a > 0) ? b : (S)0;   // 14: ifpos
    }
}

constexpr int kNumBinops = 15;

// A[i] = op(A[i], B[idx[i]])  (idx = per-nonzero column for sdoprow, row for
// sdopcol); with idx == nullptr every nonzero uses B[0].
template <typename S>
__global__ void __launch_bounds__(kThreads)
sdop_kernel(long long nnz, S *__restrict__ A, const int *__restrict__ idx, const S *__restrict__ B, int opn) {
    const long long stride = (long long)gridDim.x * kThreads;
    for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < nnz; i += stride) {
        const S b = idx ? __ldg(B + __ldg(idx + i)) : __ldg(B);
        A[i] = apply_binop<S>(opn, A[i], b);
    }
}

// ---------------------------------------------------------------------------
// Segmented sum:  B[seg[j]] += P[j]  for a non-decreasing seg, streaming 8 (or 12)
// bytes per nonzero.  One warp takes a chunk of 32*ITEMS consecutive nonzeros, reads
// it in ITEMS coalesced rows and sums each run of equal segments with a segmented
// warp scan (a fixed tree order: bit-reproducible).  A run that lies inside the chunk
// is added to B by the one lane holding its last element (plain load/add/store: no
// other lane or warp owns that entry).  A run that crosses a chunk boundary is
// stored as a piece in the same two-slots-per-chunk layout the gather-accumulate
// kernel uses, and ga_fixup_kernel with k = 1 adds the pieces in chunk order.
// ---------------------------------------------------------------------------
template <typename S, int ITEMS>
__global__ void __launch_bounds__(kThreads)
segsum_chunk_kernel(long long nnz, long long nchunks, const S *__restrict__ P, const int *__restrict__ seg,
                    S *__restrict__ B, S *__restrict__ part) {
    constexpr int CHUNK = 32 * ITEMS;
    const int lane = threadIdx.x & 31;
    const long long c = ((long long)blockIdx.x * kThreads + threadIdx.x) >> 5;
    if (c >= nchunks) return;
    const long long j0 = c * CHUNK;
    const long long j1 = (j0 + CHUNK < nnz) ? j0 + CHUNK : nnz;
    // everything the chunk needs is loaded first (ITEMS independent coalesced rows of keys and
    // values, plus the two keys either side of the chunk), then summed from registers
    int key[ITEMS];
    S val[ITEMS];
    const int last_key = __ldg(seg + j1 - 1);
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const long long j = j0 + (long long)i * 32 + lane;
        const bool valid = j < j1;
        // padding lanes get a key of their own (no segment contains them) and add nothing
        key[i] = valid ? __ldg(seg + j) : ~last_key;
        val[i] = valid ? __ldg(P + j) : (S)0;
    }
    const int first = __shfl_sync(0xffffffffu, key[0], 0);
    const int before = (j0 > 0) ? __ldg(seg + j0 - 1) : ~first;
    const int after = (j1 < nnz) ? __ldg(seg + j1) : ~last_key;
    const bool head_open = before == first;
    int carry_key = first;
    S carry = 0;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const long long j = j0 + (long long)i * 32 + lane;
        const bool valid = j < j1;
        const int k_ = key[i];
        // key of the next element: the next lane's, for lane 31 lane 0 of the next row, after the chunk `after`
        int next = __shfl_down_sync(0xffffffffu, k_, 1);
        const int next_row0 = __shfl_sync(0xffffffffu, (i + 1 < ITEMS) ? key[i + 1 < ITEMS ? i + 1 : i] : after, 0);
        if (lane == 31) next = next_row0;
        if (valid && j == j1 - 1) next = after;
        S v = val[i];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const S uv = __shfl_up_sync(0xffffffffu, v, d);
            const int uk = __shfl_up_sync(0xffffffffu, k_, d);
            if (lane >= d && uk == k_) v += uv;
        }
        if (k_ == carry_key) v += carry;           // the run that came in from the previous row of this chunk
        const bool last = valid && j == j1 - 1;    // last element of the chunk
        const bool ends = valid && next != k_;     // last element of its run
        if (ends) {
            if (head_open && k_ == first) part[c * 2] = v;       // piece of the run that entered from the left
            else B[k_] += v;
        } else if (last) {
            part[c * 2 + ((head_open && k_ == first) ? 0 : 1)] = v;    // the run goes on in the next chunk
        }
        const int k31 = __shfl_sync(0xffffffffu, k_, 31);
        const S v31 = __shfl_sync(0xffffffffu, v, 31);
        const bool e31 = __shfl_sync(0xffffffffu, (int)ends, 31) != 0;
        carry_key = k31;
        carry = e31 ? (S)0 : v31;
    }
}

}  // namespace bidmat
