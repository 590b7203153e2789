// Sum of the per-GPU partial results of B*^S over NVLink peer memory.
//
// Every rank holds a full-size partial G in a buffer its peers can address.
// Rank r owns the r-th slice of the element range: it reads that slice from
// every rank's buffer with plain peer loads, adds the values in rank order
// 0..W-1 (so every GPU ends up with bit-identical sums, whatever the timing),
// and writes the total back into every rank's buffer with peer stores: a
// reduce-scatter by pulling and an all-gather by pushing in one kernel, with
// no float atomics.  The caller must make sure, with its own cross-rank
// synchronisation, that all partials are complete before the kernel starts on
// any rank and that nobody touches the buffers until it has finished on all
// ranks; the kernel itself never waits on another GPU.
#include <cuda_runtime.h>

#include "../../include/bidmat_b200.h"
#include "host_common.cuh"

using namespace bidmat;

namespace {

constexpr int kMaxPeers = 16;
struct PeerPtrs { float *p[kMaxPeers]; };

template <int W>
__global__ void __launch_bounds__(256)
peer_sum_kernel(PeerPtrs peers, long long v_begin, long long v_end) {
    // float4 index range [v_begin, v_end) of this rank's slice
    constexpr int UNROLL = (W <= 4) ? 4 : 2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long v0 = v_begin + (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < v_end; v0 += stride * UNROLL) {
        float4 x[UNROLL][W];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const long long v = v0 + u * stride;
#pragma unroll
            for (int r = 0; r < W; r++)
                x[u][r] = (v < v_end) ? reinterpret_cast<const float4 *>(peers.p[r])[v] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const long long v = v0 + u * stride;
            if (v >= v_end) continue;
            float4 s = x[u][0];
#pragma unroll
            for (int r = 1; r < W; r++) { s.x += x[u][r].x; s.y += x[u][r].y; s.z += x[u][r].z; s.w += x[u][r].w; }
#pragma unroll
            for (int r = 0; r < W; r++) reinterpret_cast<float4 *>(peers.p[r])[v] = s;
        }
    }
}

// Same sum when every rank knows which rows (columns of k floats of the k x m result)
// each rank wrote: touched[r * words + w] bit b set = rank r wrote row 32*w + b.  A
// rank's row is only read when that rank wrote it, so ranks need not clear the rows
// they did not write (they may hold anything, e.g. the previous sum), and rows that
// nobody wrote are set to zero.  Requires k % 4 == 0.
template <int W>
__global__ void __launch_bounds__(256)
peer_sum_rows_kernel(PeerPtrs peers, long long v_begin, long long v_end, int vec_per_row,
                     const unsigned *__restrict__ touched, long long words) {
    constexpr int UNROLL = (W <= 4) ? 4 : 2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long v0 = v_begin + (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < v_end; v0 += stride * UNROLL) {
        float4 x[UNROLL][W];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const long long v = v0 + u * stride;
            const long long row = (v < v_end ? v : v_begin) / vec_per_row;
            const long long w = row >> 5;
            const int bit = (int)(row & 31);
#pragma unroll
            for (int r = 0; r < W; r++) {
                const bool wrote = (__ldg(touched + r * words + w) >> bit) & 1u;
                x[u][r] = (v < v_end && wrote) ? reinterpret_cast<const float4 *>(peers.p[r])[v]
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const long long v = v0 + u * stride;
            if (v >= v_end) continue;
            float4 s = x[u][0];
#pragma unroll
            for (int r = 1; r < W; r++) { s.x += x[u][r].x; s.y += x[u][r].y; s.z += x[u][r].z; s.w += x[u][r].w; }
#pragma unroll
            for (int r = 0; r < W; r++) reinterpret_cast<float4 *>(peers.p[r])[v] = s;
        }
    }
}

// The same sum through the NVSwitch: `mc` is a multicast address that maps the buffers of
// all ranks.  multimem.ld_reduce makes the switch fetch this rank's slice from every GPU and
// add it on the way (one load instead of W, 1/W of the inbound traffic); multimem.st stores
// the total into every rank's buffer at once (one store instead of W, 1/W of the outbound
// traffic).  Per GPU and direction about half as many bytes cross NVLink as with peer loads
// and stores.  One GPU reduces each element and all receive its result, so the ranks end
// bit-identical; the order of the additions inside the switch is the hardware's.
template <int UNROLL>
__global__ void __launch_bounds__(256)
mc_sum_kernel(float *mc, long long v_begin, long long v_end) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    float4 *p = reinterpret_cast<float4 *>(mc);
    for (long long v0 = v_begin + (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < v_end; v0 += stride * UNROLL) {
        float4 x[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const long long v = v0 + u * stride;
            x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (v < v_end)
                asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(x[u].x), "=f"(x[u].y), "=f"(x[u].z), "=f"(x[u].w) : "l"(p + v) : "memory");
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const long long v = v0 + u * stride;
            if (v < v_end)
                asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                             ::"l"(p + v), "f"(x[u].x), "f"(x[u].y), "f"(x[u].z), "f"(x[u].w) : "memory");
        }
    }
}

int peer_args(int world, int rank, const unsigned long long *peer_addresses, long long count, PeerPtrs *pp,
              long long *v_begin, long long *v_end) {
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || count < 0 || !peer_addresses)
        return (int)cudaErrorInvalidValue;
    if (count % 4 != 0) return (int)cudaErrorInvalidValue;
    for (int r = 0; r < kMaxPeers; r++) pp->p[r] = nullptr;
    for (int r = 0; r < world; r++) {
        if (peer_addresses[r] == 0 || (peer_addresses[r] & 15ull)) return (int)cudaErrorInvalidValue;
        pp->p[r] = reinterpret_cast<float *>(peer_addresses[r]);
    }
    const long long nvec = count / 4;
    const long long per = (nvec + world - 1) / world;
    *v_begin = per * rank < nvec ? per * rank : nvec;
    *v_end = *v_begin + per < nvec ? *v_begin + per : nvec;
    return 0;
}

}  // namespace

extern "C" int bidmat_b200_mc_allreduce_sum_range(int world, int rank, void *multicast_address, long long first,
                                                  long long count, int ctas, bidmat_stream_t stream) {
    if (world < 1 || rank < 0 || rank >= world || first < 0 || first % 4 != 0 || count < 0 || count % 4 != 0 ||
        !multicast_address || (reinterpret_cast<uintptr_t>(multicast_address) & 15u))
        return (int)cudaErrorInvalidValue;
    if (count == 0 || world == 1) return 0;
    // the 16-byte vectors of the range, cut into `world` slices: this rank reduces slice `rank`
    const long long nvec = count / 4;
    const long long per = (nvec + world - 1) / world;
    long long v_begin = per * rank < nvec ? per * rank : nvec;
    long long v_end = v_begin + per < nvec ? v_begin + per : nvec;
    if (v_end <= v_begin) return 0;
    v_begin += first / 4;
    v_end += first / 4;
    if (ctas <= 0) ctas = (world >= 8) ? 96 : 64;     // measured on 8 GPUs: 32 CTAs leave 0.8 ms of the sum exposed, 96 none
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : cudaStreamPerThread;
    // 16-byte reductions in flight per thread: BIDMAT_B200_MC_UNROLL = 4 (default), 8 or 16
    const int unroll = env_int("BIDMAT_B200_MC_UNROLL", 4);
    float *mc = static_cast<float *>(multicast_address);
    if (unroll >= 16) mc_sum_kernel<16><<<ctas, 256, 0, st>>>(mc, v_begin, v_end);
    else if (unroll >= 8) mc_sum_kernel<8><<<ctas, 256, 0, st>>>(mc, v_begin, v_end);
    else mc_sum_kernel<4><<<ctas, 256, 0, st>>>(mc, v_begin, v_end);
    g_launches += 1;
    return (int)cudaGetLastError();
}

extern "C" int bidmat_b200_mc_allreduce_sum(int world, int rank, void *multicast_address, long long count, int ctas,
                                            bidmat_stream_t stream) {
    return bidmat_b200_mc_allreduce_sum_range(world, rank, multicast_address, 0, count, ctas, stream);
}

extern "C" int bidmat_b200_peer_allreduce_sum_rows_range(int world, int rank, const unsigned long long *peer_addresses,
                                                         int k, long long m, const unsigned *touched,
                                                         long long row_begin, long long row_end, int ctas,
                                                         bidmat_stream_t stream) {
    if (k <= 0 || k % 4 != 0 || m < 0 || !touched || row_begin < 0 || row_end > m || row_begin > row_end)
        return (int)cudaErrorInvalidValue;
    PeerPtrs pp;
    long long v_begin = 0, v_end = 0;
    // the float4 elements of the row range, cut into `world` slices like a whole buffer
    const int bad = peer_args(world, rank, peer_addresses, (long long)k * (row_end - row_begin), &pp, &v_begin, &v_end);
    if (bad) return bad;
    if (row_end == row_begin || world == 1 || v_end <= v_begin) return 0;
    const long long v0 = row_begin * (long long)(k / 4);
    v_begin += v0;
    v_end += v0;
    if (ctas <= 0) ctas = (world <= 2) ? 64 : 48;      // measured on 8 GPUs: 32 leave 0.9 ms of the sum exposed, 48 leave 0.4
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : cudaStreamPerThread;
    const long long words = (m + 31) / 32;
    switch (world) {
        case 2: peer_sum_rows_kernel<2><<<ctas, 256, 0, st>>>(pp, v_begin, v_end, k / 4, touched, words); break;
        case 4: peer_sum_rows_kernel<4><<<ctas, 256, 0, st>>>(pp, v_begin, v_end, k / 4, touched, words); break;
        case 8: peer_sum_rows_kernel<8><<<ctas, 256, 0, st>>>(pp, v_begin, v_end, k / 4, touched, words); break;
        default: return (int)cudaErrorInvalidValue;
    }
    g_launches += 1;
    return (int)cudaGetLastError();
}

extern "C" int bidmat_b200_peer_allreduce_sum_rows(int world, int rank, const unsigned long long *peer_addresses,
                                                   int k, long long m, const unsigned *touched, int ctas,
                                                   bidmat_stream_t stream) {
    return bidmat_b200_peer_allreduce_sum_rows_range(world, rank, peer_addresses, k, m, touched, 0, m, ctas, stream);
}

extern "C" int bidmat_b200_peer_allreduce_sum(int world, int rank, const unsigned long long *peer_addresses,
                                              long long count, int ctas, bidmat_stream_t stream) {
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || count < 0 || !peer_addresses)
        return (int)cudaErrorInvalidValue;
    if (count == 0 || world == 1) return 0;
    if (count % 4 != 0) return (int)cudaErrorInvalidValue;
    PeerPtrs pp;
    for (int r = 0; r < kMaxPeers; r++) pp.p[r] = nullptr;
    for (int r = 0; r < world; r++) {
        if (peer_addresses[r] == 0 || (peer_addresses[r] & 15ull)) return (int)cudaErrorInvalidValue;
        pp.p[r] = reinterpret_cast<float *>(peer_addresses[r]);
    }
    const long long nvec = count / 4;
    const long long per = (nvec + world - 1) / world;
    const long long v_begin = per * rank < nvec ? per * rank : nvec;
    const long long v_end = v_begin + per < nvec ? v_begin + per : nvec;
    if (v_end <= v_begin) return 0;
    // Default CTA count: enough to finish underneath A*S and DDS, which shrink with the
    // number of GPUs, without taking many SMs from them (measured on 8 GPUs: 16 leave the
    // sum exposed, 64 slow the products; on 2 GPUs 32 leave it exposed, 64 hide it).
    if (ctas <= 0) ctas = (world <= 2) ? 64 : (world <= 4) ? 48 : 32;
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : cudaStreamPerThread;
    switch (world) {
        case 2: peer_sum_kernel<2><<<ctas, 256, 0, st>>>(pp, v_begin, v_end); break;
        case 4: peer_sum_kernel<4><<<ctas, 256, 0, st>>>(pp, v_begin, v_end); break;
        case 8: peer_sum_kernel<8><<<ctas, 256, 0, st>>>(pp, v_begin, v_end); break;
        default: return (int)cudaErrorInvalidValue;   // one process per GPU of a 2-, 4- or 8-GPU box
    }
    g_launches += 1;
    return (int)cudaGetLastError();
}
