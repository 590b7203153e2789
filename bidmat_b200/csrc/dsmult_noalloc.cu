// A*S for callers that must not allocate device memory.
//
// bidmat_b200_dsmult_noalloc computes the same C += A * S as
// bidmat_b200_dsmult_async, with the same gather-accumulate and fix-up kernels,
// but its scratch (the partial sums of columns that straddle two chunks of the
// nonzero list) lives in the fixed array below instead of the library's
// growable workspace.  The call makes no cudaMalloc, cudaFree, event or stream
// creation and uses no allocating library routine.
//
// Who needs this: a host application that hands all device memory to its own
// caching allocator (BIDMat's GPU cache does, and so does a PyTorch process
// that has filled its pool), where a cudaMalloc issued from inside a library
// can fail or fragment the pool; and a multi-stream serving loop, where the
// device-wide synchronisation implied by cudaMalloc/cudaFree would stall
// every other stream.
//
// The array is one per device and is shared by every call on that device.  It
// keeps whatever the previous call left in it; that is harmless here because
// each slot the fix-up kernel reads is written earlier in the same call by the
// chunk kernel (nothing has to start at zero).  Two calls that overlap on the
// GPU (different streams, or different host threads on the same device) race
// on the array and give wrong sums: order them on one stream or with events.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/bidmat_b200.h"
#include "kernels.cuh"
#include "host_common.cuh"

using namespace bidmat;

namespace {

// 16 MiB of device memory on every GPU that loads the library, until exit.
static __device__ __align__(256) float g_noalloc_scratch[BIDMAT_B200_NOALLOC_SCRATCH_FLOATS];

// Device address of g_noalloc_scratch per device.  In host code the array's
// name is only a handle for cudaGetSymbolAddress, never a device pointer.
std::mutex g_addr_mu;
float *g_scratch_addr[64] = {nullptr};

// Resolves the array's device address for the current device (first call per
// device; later calls read the cached pointer).
cudaError_t scratch_for_current_device(float **out) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(g_addr_mu);
    if (g_scratch_addr[dev] == nullptr) {
        float *ptr = nullptr;
        err = cudaGetSymbolAddress((void **)&ptr, g_noalloc_scratch);
        if (err != cudaSuccess) return err;
        if (ptr == nullptr) return cudaErrorInvalidSymbol;
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return cudaSuccess;
}

}  // namespace

extern "C" int bidmat_b200_dsmult_noalloc(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                                          const int *Bir, const int *Bic, float *C, bidmat_stream_t stream) {
    if (nrows < 0 || ncols < 0 || nnz < 0) return (int)cudaErrorInvalidValue;
    if (nnz == 0 || nrows == 0) return 0;
    if (!A || !Bdata || !Bir || !Bic || !C) return (int)cudaErrorInvalidValue;

    // Chunk length: the usual choice, lengthened until 2*nrows floats per chunk
    // fit the fixed array; beyond BIDMAT_B200_NOALLOC_MAX_CHUNK the problem is
    // too large for this entry point and is rejected before anything is launched.
    const Shape s = pick_shape(nrows, is16(A) && is16(C));
    const long long max_chunks = (long long)BIDMAT_B200_NOALLOC_SCRATCH_FLOATS / (2LL * nrows);
    if (max_chunks < 1) return (int)cudaErrorInvalidValue;
    long long chunk = pick_chunk(nnz, s.lpv);
    const long long fit = (nnz + max_chunks - 1) / max_chunks;
    if (chunk < fit) chunk = ((fit + s.lpv - 1) / s.lpv) * s.lpv;
    if (chunk > BIDMAT_B200_NOALLOC_MAX_CHUNK) return (int)cudaErrorInvalidValue;
    const long long nchunks = (nnz + chunk - 1) / chunk;
    if (ga_part_floats(nrows, nnz, (int)chunk) > (size_t)BIDMAT_B200_NOALLOC_SCRATCH_FLOATS)
        return (int)cudaErrorInvalidValue;

    float *part = nullptr;
    cudaError_t err = scratch_for_current_device(&part);
    if (err != cudaSuccess) return (int)err;

    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : cudaStreamPerThread;
    dim3 grid(blocks_for(nchunks, s.lpv), s.tiles, 1);
    const int ichunk = (int)chunk;
    constexpr int kWideVec = 4;
    // Dense heights 32..512 with 16-byte aligned operands take the same predicate-free
    // gather kernel as bidmat_b200_dsmult_async (it needs nothing but `part` either).
    if (s.vec == 4 && s.tiles == 1 && nrows == 4 * s.lpv * s.nt && !env_int("BIDMAT_B200_GENERIC", 0)) {
        constexpr int kFast = 128;
        const int wpb = kFast / s.lpv;
        dim3 fgrid((unsigned)((nchunks + wpb - 1) / wpb), 1, 1);
#define CALL_FAST_NOALLOC(LPV, NT, U, MINB)                                                             \
    ga_chunk_fast_kernel<float, LPV, NT, U, kFast, MINB><<<fgrid, kFast, 0, st>>>(nnz, ichunk, nchunks, A, Bdata, Bir, Bic, C, \
                                                                        part, nullptr, 0xffffffffu)
        if (s.lpv == 8) CALL_FAST_NOALLOC(8, 1, 4, 0);
        else if (s.lpv == 16) CALL_FAST_NOALLOC(16, 1, 4, 0);
        else if (s.nt == 1) CALL_FAST_NOALLOC(32, 1, 4, 0);
        else if (s.nt == 2) CALL_FAST_NOALLOC(32, 2, 2, 5);
        else CALL_FAST_NOALLOC(32, 4, 1, 0);
#undef CALL_FAST_NOALLOC
        if (nchunks > 1) {
#define CALL_FIX_NOALLOC(VEC, LPV, NT)                                                                  \
    ga_fixup_kernel<float, VEC, LPV, NT><<<grid, kThreads, 0, st>>>(nrows, nnz, ichunk, nchunks, Bic, C, part, nullptr, \
                                                                    0xffffffffu, nrows);
            DISPATCH_SHAPE(s, CALL_FIX_NOALLOC);
#undef CALL_FIX_NOALLOC
        }
        g_launches += (nchunks > 1) ? 2 : 1;
        return (int)cudaGetLastError();
    }
#define CALL_GA_NOALLOC(VEC, LPV, NT)                                                                  \
    ga_chunk_kernel<float, VEC, LPV, NT, 4><<<grid, kThreads, 0, st>>>(nrows, nnz, ichunk, nchunks, A, Bdata, \
                                                                Bir, Bic, C, part, nullptr,           \
                                                                0xffffffffu, nrows, nrows, nullptr, 0u); \
    if (nchunks > 1)                                                                                   \
        ga_fixup_kernel<float, VEC, LPV, NT><<<grid, kThreads, 0, st>>>(nrows, nnz, ichunk, nchunks, Bic, C, part, nullptr, \
                                                                        0xffffffffu, nrows);
    DISPATCH_SHAPE(s, CALL_GA_NOALLOC);
#undef CALL_GA_NOALLOC
    g_launches += (nchunks > 1) ? 2 : 1;
    return (int)cudaGetLastError();
}
