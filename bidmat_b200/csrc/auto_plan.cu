// Prepared structures behind the reference-signature B*^S entry points.
//
// BIDMat's native signature (CUMAT.dsmultT, CUMAT.java:152) carries nothing but
// arrays, so bidmat_b200_dsmultT has to order the nonzeros by row on every call.
// A BIDMat process multiplies with the same structure again and again (every
// G = B *^ DDS(A,B,S) of a factorisation loop has S's pattern), and a binding that
// only rebinds the natives cannot create a plan handle itself.  When switched on
// (bidmat_b200_set_auto_plan(1) or BIDMAT_B200_AUTO_PLAN=1), the synchronous entry
// points do it for the caller:
//   * every call first takes a 128-bit fingerprint of (Bir, Bic) and the largest row
//     index in one coalesced pass over the two index arrays (about the time of a copy
//     of them) and reads it back;
//   * a structure seen for the second time gets a plan (built once, kept by the
//     library, at most kMaxPlans per GPU, least recently used first out; structures
//     that come by once, like the minibatches of a streaming pass, never cost a plan
//     and never push one out);
//   * a call whose sizes, dense height, element type and fingerprint equal those of
//     a kept plan runs through it: no sort, the predicate-free plan kernels;
//   * anything else takes the ordinary path.
// The match is by fingerprint, not by comparing the arrays: two different
// structures of the same size collide with probability 2^-128.  Pointers are never
// part of the key (BIDMat recycles its buffers, GSMat.scala:234-248).  Off by
// default because a kept plan holds about 13 bytes per nonzero of device memory
// that the host application does not see.
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "../../include/bidmat_b200.h"
#include "auto_plan.cuh"
#include "host_common.cuh"
#include "workspace.cuh"

namespace bidmat {
namespace {

constexpr int kMaxPlans = 2;      // plans kept per GPU
constexpr int kMaxSeen = 8;       // structures remembered after one sighting, without a plan

struct Fingerprint {
    unsigned long long h1 = 0, h2 = 0;
    int maxrow = -1;
    bool same(const Fingerprint &o) const { return h1 == o.h1 && h2 == o.h2 && maxrow == o.maxrow; }
};

struct Entry {
    bidmat_b200_plan_t plan = nullptr;   // null: the structure has been seen once, no plan yet
    int nnz = 0, ncols = 0, k = 0, elem = 0;
    Fingerprint fp;
    unsigned long long stamp = 0;
};

struct DeviceCache {
    std::mutex mu;                           // held for the whole call: calls on one GPU take turns
    std::vector<Entry> entries;
    unsigned long long clock = 0;
    unsigned long long *dev_out = nullptr;   // {h1, h2, maxrow} on the device
};

DeviceCache g_cache[kMaxDevices];
std::atomic<int> g_enabled{-1};              // -1: not decided yet (environment)
std::atomic<long long> g_built{0}, g_planned_calls{0}, g_plain_calls{0};

__device__ __forceinline__ unsigned long long mix64(unsigned long long x, unsigned long long c1, unsigned long long c2) {
    x ^= x >> 30; x *= c1;
    x ^= x >> 27; x *= c2;
    x ^= x >> 31;
    return x;
}

// out[0], out[1] += two independent 64-bit hashes of (position, row, column), summed over
// the nonzeros (integer sums: the order does not matter); out[2] = max row.
__global__ void __launch_bounds__(256)
fingerprint_kernel(long long n, const int *__restrict__ ir, const int *__restrict__ ic, unsigned long long *out) {
    unsigned long long s1 = 0, s2 = 0;
    int mx = -1;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) {
        const int r = __ldg(ir + j), c = __ldg(ic + j);
        const unsigned long long x = (((unsigned long long)(unsigned)r) << 32 | (unsigned)c) +
                                     (unsigned long long)j * 0x9E3779B97F4A7C15ull;
        s1 += mix64(x, 0xBF58476D1CE4E5B9ull, 0x94D049BB133111EBull);
        s2 += mix64(x ^ 0xD6E8FEB86659FD93ull, 0xFF51AFD7ED558CCDull, 0xC4CEB9FE1A85EC53ull);
        mx = r > mx ? r : mx;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
        const int t = __shfl_xor_sync(0xffffffffu, mx, o);
        mx = t > mx ? t : mx;
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(out, s1);
        atomicAdd(out + 1, s2);
        atomicMax(reinterpret_cast<long long *>(out + 2), (long long)mx);
    }
}

bool enabled() {
    int v = g_enabled.load();
    if (v < 0) {
        v = env_int("BIDMAT_B200_AUTO_PLAN", 0) ? 1 : 0;
        int expected = -1;
        g_enabled.compare_exchange_strong(expected, v);
        v = g_enabled.load();
    }
    return v == 1;
}

void drop_all() {
    for (int d = 0; d < kMaxDevices; d++) {
        std::lock_guard<std::mutex> lock(g_cache[d].mu);
        for (Entry &e : g_cache[d].entries)
            if (e.plan) bidmat_b200_plan_destroy(e.plan);
        g_cache[d].entries.clear();
    }
}

}  // namespace

// Tries to run C += A * B^T through a kept plan.  *handled = 1: done (the return value is
// the call's status, the stream is synchronised); *handled = 0: the caller takes the
// ordinary path, with *m_seen = number of rows the index array names (0 if unknown).
int auto_plan_dsmultT(int elem, int k, int ncols, int nnz, const void *A, const void *Bdata, const int *Bir,
                      const int *Bic, void *C, int *handled, int *m_seen) {
    *handled = 0;
    *m_seen = 0;
    if (!enabled() || nnz <= 0 || k <= 0 || ncols <= 0 || !A || !Bdata || !Bir || !Bic || !C) return 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    DeviceCache &dc = g_cache[dev];
    std::lock_guard<std::mutex> lock(dc.mu);
    cudaStream_t st = cudaStreamPerThread;
    if (!dc.dev_out && cudaMalloc(&dc.dev_out, 3 * sizeof(unsigned long long)) != cudaSuccess) {
        dc.dev_out = nullptr;
        cudaGetLastError();
        return 0;
    }
    const long long init[3] = {0, 0, -1};
    unsigned long long host[3];
    cudaError_t err = cudaMemcpyAsync(dc.dev_out, init, sizeof(init), cudaMemcpyHostToDevice, st);
    if (err != cudaSuccess) return (int)err;
    fingerprint_kernel<<<148 * 8, 256, 0, st>>>((long long)nnz, Bir, Bic, dc.dev_out);
    g_launches += 1;
    err = cudaMemcpyAsync(host, dc.dev_out, sizeof(host), cudaMemcpyDeviceToHost, st);
    if (err == cudaSuccess) err = cudaStreamSynchronize(st);
    if (err != cudaSuccess) return (int)err;
    Fingerprint fp;
    fp.h1 = host[0];
    fp.h2 = host[1];
    fp.maxrow = (int)(long long)host[2];
    if (fp.maxrow < 0) return 0;                       // negative rows: let the ordinary path refuse them
    *m_seen = fp.maxrow + 1;

    Entry *hit = nullptr;
    for (Entry &e : dc.entries)
        if (e.nnz == nnz && e.ncols == ncols && e.k == k && e.elem == elem && e.fp.same(fp)) hit = &e;
    // the least recently used entry with (want_plan) or without a plan, -1 if there are fewer than `cap`
    auto oldest_of = [&](bool want_plan, int cap) {
        int count = 0, oldest = -1;
        for (size_t i = 0; i < dc.entries.size(); i++) {
            if ((dc.entries[i].plan != nullptr) != want_plan) continue;
            count++;
            if (oldest < 0 || dc.entries[i].stamp < dc.entries[(size_t)oldest].stamp) oldest = (int)i;
        }
        return count >= cap ? oldest : -1;
    };
    if (!hit) {
        // first sight of this structure (at this height): remember it, no plan yet
        const int drop = oldest_of(false, kMaxSeen);
        if (drop >= 0) dc.entries.erase(dc.entries.begin() + drop);
        Entry e;
        e.nnz = nnz; e.ncols = ncols; e.k = k; e.elem = elem; e.fp = fp; e.stamp = ++dc.clock;
        dc.entries.push_back(e);
        g_plain_calls++;
        return 0;
    }
    hit->stamp = ++dc.clock;
    if (!hit->plan) {
        const int drop = oldest_of(true, kMaxPlans);
        if (drop >= 0) {
            bidmat_b200_plan_destroy(dc.entries[(size_t)drop].plan);
            const size_t hit_index = (size_t)(hit - dc.entries.data());
            dc.entries.erase(dc.entries.begin() + drop);
            hit = &dc.entries[hit_index > (size_t)drop ? hit_index - 1 : hit_index];
        }
        bidmat_b200_plan_t p = nullptr;
        const int rc = bidmat_b200_dsmultT_plan_create(k, ncols, nnz, fp.maxrow + 1, Bir, Bic, elem, st, &p);
        if (rc != 0) {                                  // e.g. no memory for it: the ordinary path still works
            cudaGetLastError();
            g_plain_calls++;
            return 0;
        }
        hit->plan = p;
        g_built++;
    }
    int rc;
    if (elem == 4)
        rc = bidmat_b200_dsmultT_planned(hit->plan, k, ncols, nnz, static_cast<const float *>(A),
                                         static_cast<const float *>(Bdata), static_cast<float *>(C), 0, st);
    else
        rc = bidmat_b200_dsmultT_planned_f64(hit->plan, k, ncols, nnz, static_cast<const double *>(A),
                                             static_cast<const double *>(Bdata), static_cast<double *>(C), 0, st);
    *handled = 1;
    g_planned_calls++;
    return finish_sync((cudaError_t)rc, st);
}

}  // namespace bidmat

extern "C" int bidmat_b200_set_auto_plan(int enable) {
    bidmat::g_enabled.store(enable ? 1 : 0);
    if (!enable) bidmat::drop_all();
    return 0;
}

extern "C" int bidmat_b200_auto_plan_info(long long *out, int count) {
    if (!out || count < 0) return (int)cudaErrorInvalidValue;
    long long kept = 0, bytes = 0;
    for (int d = 0; d < bidmat::kMaxDevices; d++) {
        std::lock_guard<std::mutex> lock(bidmat::g_cache[d].mu);
        for (const bidmat::Entry &e : bidmat::g_cache[d].entries)
            if (e.plan) {
                long long info[BIDMAT_B200_PLAN_INFO_COUNT] = {0};
                bidmat_b200_plan_info(e.plan, info, BIDMAT_B200_PLAN_INFO_COUNT);
                kept++;
                bytes += info[11];
            }
    }
    const long long v[6] = {bidmat::enabled() ? 1 : 0, bidmat::g_built.load(), bidmat::g_planned_calls.load(),
                            bidmat::g_plain_calls.load(), kept, bytes};
    for (int i = 0; i < count && i < 6; i++) out[i] = v[i];
    return 0;
}
