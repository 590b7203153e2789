// Small structure kernels around the path: column pointers <-> per-nonzero
// columns, structure validation, permutation gathers.  Included by exactly one
// translation unit (they are ordinary, non-template kernels).
#pragma once
#include "common.cuh"

namespace bidmat {

// ---------------------------------------------------------------------------
// Structure helpers
// ---------------------------------------------------------------------------

// ic[j] = column of nonzero j, by binary search in jc (largest c with jc[c] <= j,
// skipping empty columns).
__global__ void __launch_bounds__(kThreads)
expand_jc_kernel(int ncols, long long nnz, const int *__restrict__ jc, int *__restrict__ ic) {
    const long long j = (long long)blockIdx.x * kThreads + threadIdx.x;
    if (j >= nnz) return;
    int lo = 0, hi = ncols;  // invariant: jc[lo] <= j < jc[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((long long)__ldg(jc + mid) <= j) lo = mid; else hi = mid;
    }
    ic[j] = lo;
}

// jc[c] = first j with ic[j] >= c.  Thread j fills the pointers of the columns
// in (ic[j-1], ic[j]]; the thread of the last nonzero also fills the tail.
__global__ void __launch_bounds__(kThreads)
compress_ic_kernel(int ncols, long long nnz, const int *__restrict__ ic, int *__restrict__ jc) {
    const long long j = (long long)blockIdx.x * kThreads + threadIdx.x;
    if (nnz == 0) {
        if (j <= ncols) jc[j] = 0;
        return;
    }
    if (j >= nnz) return;
    const int cj = __ldg(ic + j);
    const int prev = (j == 0) ? -1 : __ldg(ic + j - 1);
    for (int c = prev + 1; c <= cj && c <= ncols; c++) jc[c] = (int)j;
    if (j == nnz - 1)
        for (int c = cj + 1; c <= ncols; c++) jc[c] = (int)nnz;
}

// flags[0] |= 1 if a row index is outside [0, m); |= 2 if a column index is
// outside [0, ncols); |= 4 if ic decreases somewhere.
__global__ void __launch_bounds__(kThreads)
check_structure_kernel(int m, int ncols, long long nnz, const int *__restrict__ ir,
                       const int *__restrict__ ic, int *__restrict__ flags) {
    const long long j = (long long)blockIdx.x * kThreads + threadIdx.x;
    if (j >= nnz) return;
    int bad = 0;
    const int r = __ldg(ir + j), c = __ldg(ic + j);
    if (r < 0 || r >= m) bad |= 1;
    if (c < 0 || c >= ncols) bad |= 2;
    if (j > 0 && __ldg(ic + j - 1) > c) bad |= 4;
    if (bad) atomicOr(flags, bad);
}

// gathered copies through a permutation: oi[p] = ii[perm[p]], of[p] = fi[perm[p]]
__global__ void __launch_bounds__(kThreads)
permute_pairs_kernel(long long nnz, const int *__restrict__ perm, const int *__restrict__ ii,
                     const float *__restrict__ fi, int *__restrict__ oi, float *__restrict__ of) {
    const long long p = (long long)blockIdx.x * kThreads + threadIdx.x;
    if (p >= nnz) return;
    const int j = __ldg(perm + p);
    oi[p] = __ldg(ii + j);
    of[p] = __ldg(fi + j);
}

__global__ void __launch_bounds__(kThreads) iota_kernel(long long n, int *__restrict__ out) {
    const long long i = (long long)blockIdx.x * kThreads + threadIdx.x;
    if (i < n) out[i] = (int)i;
}

}  // namespace bidmat
