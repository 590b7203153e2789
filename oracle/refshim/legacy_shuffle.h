/*
 * TEST INFRASTRUCTURE.  Force-included when the reference's jni/src/Arith.cu is
 * compiled for sm_100a by oracle/build.py.  The reference calls the pre-Volta
 * warp shuffles (__shfl_down, __shfl: Arith.cu:303, 325-330), which CUDA 12
 * no longer declares for this architecture.  They are mapped onto the _sync
 * forms over the lanes that are converged at the call, which is what the old
 * intrinsics meant.  Nothing else of the reference source is altered.
 */
#pragma once
#include <cuda_runtime.h>

template <typename T> __device__ __forceinline__ T __shfl_down(T v, int d) {
    return __shfl_down_sync(__activemask(), v, d);
}
template <typename T> __device__ __forceinline__ T __shfl_up(T v, int d) {
    return __shfl_up_sync(__activemask(), v, d);
}
template <typename T> __device__ __forceinline__ T __shfl_xor(T v, int d) {
    return __shfl_xor_sync(__activemask(), v, d);
}
template <typename T> __device__ __forceinline__ T __shfl(T v, int lane) {
    return __shfl_sync(__activemask(), v, lane);
}
