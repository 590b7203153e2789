// Edge operations on the values of a GSMat that sit either side of DDS in
// factorisation loops: value <- op(value, vector[row or column]), and the sums of
// the values over rows or columns.  Included by one translation unit only.
#pragma once
#include <cstdint>
#include <type_traits>
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
// bytes per nonzero.  One warp takes a chunk of 32*ITEMS consecutive nonzeros; lane l
// owns the ITEMS consecutive ones starting at j0 + l*ITEMS (16-byte loads) and walks
// them serially: a run of equal segments that lies inside the lane's piece is added
// to B at once (segments are sorted, so nobody else holds an element of it); the
// sum of the lane's first run (`head`) and of its last run (`tail`) may belong to
// runs shared with the neighbouring lanes and are combined by ONE segmented warp
// scan per chunk, in lane order (a fixed order: bit-reproducible).  A run that
// crosses a chunk boundary is stored as a piece in the two-slots-per-chunk layout of
// the gather-accumulate kernel, and ga_fixup_kernel with k = 1 adds the pieces in
// chunk order.  No float atomics.
// ---------------------------------------------------------------------------
template <typename S, int ITEMS>
__global__ void __launch_bounds__(kThreads)
segsum_chunk_kernel(long long nnz, long long nchunks, const S *__restrict__ P, const int *__restrict__ seg,
                    S *__restrict__ B, S *__restrict__ part) {
    constexpr int CHUNK = 32 * ITEMS;
    static_assert(ITEMS % 4 == 0, "a lane loads its keys as int4");
    const unsigned full = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const long long c = ((long long)blockIdx.x * kThreads + threadIdx.x) >> 5;
    if (c >= nchunks) return;
    const long long j0 = c * CHUNK;
    const long long j1 = (j0 + CHUNK < nnz) ? j0 + CHUNK : nnz;
    const long long mine = j0 + (long long)lane * ITEMS;     // this lane's first nonzero
    const int last_key = __ldg(seg + j1 - 1);
    const int first = __ldg(seg + j0);
    const int before = (j0 > 0) ? __ldg(seg + j0 - 1) : ~first;
    const int after = (j1 < nnz) ? __ldg(seg + j1) : ~last_key;
    const bool head_open = before == first;                  // the chunk's first run began in an earlier chunk

    int key[ITEMS];
    S val[ITEMS];
    // a full piece with 16-byte aligned addresses is loaded as vectors; the last chunk and odd bases by element
    const bool vec_ok = (mine + ITEMS <= j1) && (((uintptr_t)(seg + mine)) & 15u) == 0 &&
                        (((uintptr_t)(P + mine)) & 15u) == 0;
    if (vec_ok) {
        const int4 *kp = reinterpret_cast<const int4 *>(seg + mine);
#pragma unroll
        for (int q = 0; q < ITEMS / 4; q++) {
            const int4 t = __ldg(kp + q);
            key[4 * q] = t.x; key[4 * q + 1] = t.y; key[4 * q + 2] = t.z; key[4 * q + 3] = t.w;
        }
        constexpr int PER = 16 / (int)sizeof(S);
        typedef typename std::conditional<sizeof(S) == 4, float4, double2>::type PV;
        const PV *vp = reinterpret_cast<const PV *>(P + mine);
#pragma unroll
        for (int q = 0; q < ITEMS / PER; q++) {
            const PV t = __ldg(vp + q);
            const S *ts = reinterpret_cast<const S *>(&t);
#pragma unroll
            for (int e = 0; e < PER; e++) val[PER * q + e] = ts[e];
        }
    } else {
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const long long j = mine + i;
            const bool valid = j < j1;
            // padding gets a key no segment has and adds nothing
            key[i] = valid ? __ldg(seg + j) : ~last_key;
            val[i] = valid ? __ldg(P + j) : (S)0;
        }
    }

    // serial walk: interior runs go to B, the first and the last run of the piece are kept
    const int hk = key[0];
    S head = 0, run = val[0];
    bool in_head = true;
#pragma unroll
    for (int i = 1; i < ITEMS; i++) {
        if (key[i] != key[i - 1]) {
            if (in_head) { head = run; in_head = false; }
            else if (key[i - 1] != ~last_key) B[key[i - 1]] += run;
            run = val[i];
        } else {
            run += val[i];
        }
    }
    const int tk = key[ITEMS - 1];
    const bool whole = in_head;          // the piece is a single run: `run` is its sum, head and tail coincide
    const S tail = run;

    // chain[l] = sum of the run that ends lane l's piece, over all the lanes it spans so far
    const int prev_tk = __shfl_up_sync(full, tk, 1);
    const bool linked = lane > 0 && whole && prev_tk == hk;       // the whole piece continues the previous lane's run
    S chain = tail;
    bool open = linked;                  // the partial sum still wants the lanes further left
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const S up = __shfl_up_sync(full, chain, d);
        const int up_open = __shfl_up_sync(full, (int)open, d);
        if (lane >= d && open) {
            chain = up + chain;          // left part first: lane order
            open = up_open != 0;
        }
    }
    const S left = __shfl_up_sync(full, chain, 1);
    const int next_hk = __shfl_down_sync(full, hk, 1);
    const bool padded = tk == ~last_key;

    // the first run of a piece that holds further runs ends inside this lane
    if (!whole) {
        const S total = (lane > 0 && prev_tk == hk) ? left + head : head;
        if (head_open && hk == first) part[c * 2] = total;
        else B[hk] += total;
    }
    // the last run of the piece: finished unless the next lane (or the next chunk) continues it
    if (!padded) {
        const bool chunk_end = (lane == 31) || (mine + ITEMS >= j1);
        const bool goes_on = chunk_end ? (after == tk) : (next_hk == tk);
        if (!goes_on) {
            if (head_open && tk == first) part[c * 2] = chain;
            else B[tk] += chain;
        } else if (chunk_end) {
            part[c * 2 + ((head_open && tk == first) ? 0 : 1)] = chain;
        }
    }
}

}  // namespace bidmat
