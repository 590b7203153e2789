// Shared device helpers for the sparse-dense kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace bidmat {

// A "worker" is a group of LPV consecutive lanes of one warp (LPV in
// {8,16,32}).  Lane l of a worker owns the VEC-wide elements l, l+LPV,
// l+2*LPV, ... (NT of them) of a dense column, so a worker reads a column
// with fully coalesced 16-byte loads when VEC > 1.
// Vec<S, VEC>: VEC scalars of type S moved as one load/store (16 bytes when
// VEC > 1: float4 or double2).
template <typename S, int VEC> struct Vec;
template <> struct Vec<float, 1> {
    typedef float T;
    static __device__ __forceinline__ T zero() { return 0.f; }
    static __device__ __forceinline__ T ldg(const float *p) { return __ldg(p); }
    static __device__ __forceinline__ T ld(const float *p) { return *p; }
    static __device__ __forceinline__ void st(float *p, T v) { *p = v; }
    static __device__ __forceinline__ void fma(T &acc, float s, const T &x) { acc = fmaf(s, x, acc); }
    static __device__ __forceinline__ void add(T &acc, const T &x) { acc += x; }
    static __device__ __forceinline__ float dot(const T &a, const T &b, float acc) { return fmaf(a, b, acc); }
};
template <> struct Vec<float, 4> {
    typedef float4 T;
    static __device__ __forceinline__ T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
    static __device__ __forceinline__ T ldg(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
    static __device__ __forceinline__ T ld(const float *p) { return *reinterpret_cast<const float4 *>(p); }
    static __device__ __forceinline__ void st(float *p, T v) { *reinterpret_cast<float4 *>(p) = v; }
    static __device__ __forceinline__ void fma(T &acc, float s, const T &x) {
        acc.x = fmaf(s, x.x, acc.x); acc.y = fmaf(s, x.y, acc.y);
        acc.z = fmaf(s, x.z, acc.z); acc.w = fmaf(s, x.w, acc.w);
    }
    static __device__ __forceinline__ void add(T &acc, const T &x) {
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    static __device__ __forceinline__ float dot(const T &a, const T &b, float acc) {
        acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
        acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
        return acc;
    }
};
template <> struct Vec<double, 1> {
    typedef double T;
    static __device__ __forceinline__ T zero() { return 0.0; }
    static __device__ __forceinline__ T ldg(const double *p) { return __ldg(p); }
    static __device__ __forceinline__ T ld(const double *p) { return *p; }
    static __device__ __forceinline__ void st(double *p, T v) { *p = v; }
    static __device__ __forceinline__ void fma(T &acc, double s, const T &x) { acc = ::fma(s, x, acc); }
    static __device__ __forceinline__ void add(T &acc, const T &x) { acc += x; }
    static __device__ __forceinline__ double dot(const T &a, const T &b, double acc) { return ::fma(a, b, acc); }
};
template <> struct Vec<double, 2> {
    typedef double2 T;
    static __device__ __forceinline__ T zero() { return make_double2(0.0, 0.0); }
    static __device__ __forceinline__ T ldg(const double *p) { return __ldg(reinterpret_cast<const double2 *>(p)); }
    static __device__ __forceinline__ T ld(const double *p) { return *reinterpret_cast<const double2 *>(p); }
    static __device__ __forceinline__ void st(double *p, T v) { *reinterpret_cast<double2 *>(p) = v; }
    static __device__ __forceinline__ void fma(T &acc, double s, const T &x) {
        acc.x = ::fma(s, x.x, acc.x); acc.y = ::fma(s, x.y, acc.y);
    }
    static __device__ __forceinline__ void add(T &acc, const T &x) { acc.x += x.x; acc.y += x.y; }
    static __device__ __forceinline__ double dot(const T &a, const T &b, double acc) {
        acc = ::fma(a.x, b.x, acc); acc = ::fma(a.y, b.y, acc);
        return acc;
    }
};

// Mask of the lanes of the worker that contains the calling lane.
template <int LPV> __device__ __forceinline__ unsigned worker_mask() {
    if constexpr (LPV == 32) {
        return 0xffffffffu;
    } else {
        const unsigned lane = threadIdx.x & 31u;
        return ((1u << LPV) - 1u) << (lane & ~(unsigned)(LPV - 1));
    }
}

constexpr int kThreads = 256;  // threads per CTA for every kernel here

}  // namespace bidmat
