// Edge operations on the values of a GSMat that sit either side of DDS in
// factorisation loops: value <- op(value, vector[row or column]).  Included by
// one translation unit only.
#pragma once
#include "common.cuh"

namespace bidmat {

// BIDMat's binary operator table (jni/src/Operators.cu:86-101), by index.
__device__ __forceinline__ float apply_binop(int opn, float a, float b) {
    switch (opn) {
        case 0: return a + b;
        case 1: return a - b;
        case 2: return a * b;
        case 3: return a / b;
        case 4: return (a > b) ? 1.0f : 0.f;
        case 5: return (a < b) ? 1.0f : 0.f;
        case 6: return (a == b) ? 1.0f : 0.f;
        case 7: return (a >= b) ? 1.0f : 0.f;
        case 8: return (a <= b) ? 1.0f : 0.f;
        case 9: return (a != b) ? 1.0f : 0.f;
        case 10: return fmaxf(a, b);
        case 11: return fminf(a, b);
        case 12: return atan2f(a, b);
        case 13: return powf(a, b);
        default: return (a > 0) ? b : 0.f;   // 14: ifpos
    }
}

constexpr int kNumBinops = 15;

// A[i] = op(A[i], B[idx[i]])  (idx = per-nonzero column for sdoprow, row for
// sdopcol); with idx == nullptr every nonzero uses B[0].
__global__ void __launch_bounds__(kThreads)
sdop_kernel(long long nnz, float *__restrict__ A, const int *__restrict__ idx, const float *__restrict__ B, int opn) {
    const long long stride = (long long)gridDim.x * kThreads;
    for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < nnz; i += stride) {
        const float b = idx ? __ldg(B + __ldg(idx + i)) : __ldg(B);
        A[i] = apply_binop(opn, A[i], b);
    }
}

__global__ void fill_one_kernel(float *p) { *p = 1.0f; }

}  // namespace bidmat
