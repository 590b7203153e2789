// Host-side runtime shared by the translation units of the library: the
// per-device scratch pool, the optional per-kernel timing spans and small
// stream helpers.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/bidmat_b200.h"

namespace bidmat {

// ------------------------------------------------------------------ timing
// Optional per-kernel timing for the benchmark: when enabled, the launchers
// bracket their main kernels with CUDA events on the launching stream.
struct TimedSpan { const char *label; cudaEvent_t a, b; };
inline std::atomic<int> g_timing{0};
inline std::mutex g_span_mu;
inline std::vector<TimedSpan> g_spans;

struct ScopedSpan {
    cudaStream_t st;
    TimedSpan span{nullptr, nullptr, nullptr};
    ScopedSpan(const char *label, cudaStream_t s) : st(s) {
        if (!g_timing.load()) return;
        if (cudaEventCreate(&span.a) != cudaSuccess || cudaEventCreate(&span.b) != cudaSuccess) return;
        span.label = label;
        cudaEventRecord(span.a, st);
    }
    ~ScopedSpan() {
        if (!span.label) return;
        cudaEventRecord(span.b, st);
        std::lock_guard<std::mutex> g(g_span_mu);
        g_spans.push_back(span);
    }
};

// ------------------------------------------------------------------ scratch
// Scratch memory comes from one memory pool per device, owned by the library,
// through stream-ordered allocation: a lease is cudaMallocFromPoolAsync on the
// call's stream and cudaFreeAsync on the same stream when the launches have been
// enqueued, so nothing synchronises the device, calls on different streams never
// share a buffer, and the memory goes back to the pool before the call returns
// (it stays cached in the pool for the next call until release_workspace trims
// it).  A per-device byte limit refuses larger leases on the host, before any
// launch, with cudaErrorMemoryAllocation.
constexpr int kMaxDevices = 64;

struct DevicePool {
    std::mutex mu;
    cudaMemPool_t pool = nullptr;
    std::atomic<long long> limit{0};      // 0 = no limit
};
inline DevicePool g_pools[kMaxDevices];

inline cudaError_t device_pool(int dev, cudaMemPool_t *out) {
    DevicePool &p = g_pools[dev];
    std::lock_guard<std::mutex> g(p.mu);
    if (p.pool == nullptr) {
        cudaMemPoolProps props;
        memset(&props, 0, sizeof(props));
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        cudaError_t err = cudaMemPoolCreate(&p.pool, &props);
        if (err != cudaSuccess) { p.pool = nullptr; return err; }
        // keep freed blocks cached in the pool (reused by the next call) until trimmed
        unsigned long long keep = ~0ull;
        cudaMemPoolSetAttribute(p.pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    *out = p.pool;
    return cudaSuccess;
}

struct WorkspaceLease {
    cudaStream_t stream = nullptr;
    char *base = nullptr;
    size_t bytes = 0;
    size_t used = 0;
    cudaError_t err = cudaSuccess;

    WorkspaceLease(size_t want, cudaStream_t s) : stream(s), bytes(want) {
        int dev = 0;
        err = cudaGetDevice(&dev);
        if (err != cudaSuccess) return;
        if (dev < 0 || dev >= kMaxDevices) { err = cudaErrorInvalidDevice; return; }
        const long long lim = g_pools[dev].limit.load();
        if (lim > 0 && (long long)want > lim) { err = cudaErrorMemoryAllocation; return; }
        cudaMemPool_t pool = nullptr;
        err = device_pool(dev, &pool);
        if (err != cudaSuccess) return;
        void *p = nullptr;
        err = cudaMallocFromPoolAsync(&p, want ? want : 256, pool, stream);
        if (err != cudaSuccess) {
            (void)cudaGetLastError();      // the refusal is reported through `err`; leave no sticky state behind
            base = nullptr;
            return;
        }
        base = static_cast<char *>(p);
    }
    template <typename T> T *take(size_t count) {
        size_t off = (used + 255) & ~size_t(255);
        used = off + count * sizeof(T);
        return reinterpret_cast<T *>(base + off);
    }
    ~WorkspaceLease() {
        if (base) cudaFreeAsync(base, stream);
    }
    WorkspaceLease(const WorkspaceLease &) = delete;
    WorkspaceLease &operator=(const WorkspaceLease &) = delete;
};

inline size_t pad256(size_t b) { return (b + 255) & ~size_t(255); }

inline cudaStream_t as_stream(bidmat_stream_t s) {
    return s ? static_cast<cudaStream_t>(s) : cudaStreamPerThread;
}

inline int finish_sync(cudaError_t err, cudaStream_t st) {
    if (err != cudaSuccess) return (int)err;
    err = cudaStreamSynchronize(st);
    if (err != cudaSuccess) return (int)err;
    return (int)cudaGetLastError();
}

inline int ceil_log2(unsigned long long v) {  // smallest b with 2^b >= v (v >= 1)
    int b = 0;
    while ((1ull << b) < v) b++;
    return b;
}

}  // namespace bidmat
