// Kernels of the sparse-dense path: gather-accumulate over nonzero chunks (A*S
// and, on the row-sorted structure, B*^S), its deterministic fix-up, and the
// sampled dense-dense product.  sm_100a only; fp32 CUDA cores, no tensor cores:
// the work is a gather with 0.5 flop per byte.
#pragma once
#include "common.cuh"

namespace bidmat {

// ---------------------------------------------------------------------------
// Gather-accumulate:  O[:, seg[j]] += val[j] * D[:, gidx[j]]   for j in [0,nnz)
//
// `seg` is non-decreasing, so the nonzeros of one output column form one
// contiguous run.  The nonzero array is cut into chunks of `chunk` entries and
// each worker (LPV lanes) takes one chunk, which balances load by nonzeros
// whatever the column lengths are.  A run that lies inside one chunk is summed
// in registers and added to O by its only owner (plain load/add/store).  A run
// that crosses a chunk boundary is never added to O here: each chunk stores its
// piece of it in `part` (slot 0 of the chunk = piece of the run entering from
// the left, slot 1 = piece of the run leaving to the right) and ga_fixup_kernel
// adds the pieces in chunk order.  No float atomics anywhere, so the result is
// bit-reproducible.
//
// Dense column layout per worker: lane l holds VEC-wide elements l + t*LPV,
// t < NT, of the k-tile selected by blockIdx.y (tile width LPV*NT*VEC floats).
// ---------------------------------------------------------------------------
template <typename S, int VEC, int LPV, int NT, int U>
__global__ void __launch_bounds__(kThreads)
ga_chunk_kernel(int k, long long nnz, int chunk, long long nchunks,
                const S *__restrict__ D, const S *__restrict__ val,
                const int *__restrict__ gidx, const int *__restrict__ seg,
                S *__restrict__ O, S *__restrict__ part,
                const int *__restrict__ range, unsigned segmask, int ld_d, int ld_o,
                const int4 *__restrict__ desc, unsigned storebit) {
    // ld_d / ld_o: distance in elements between consecutive columns of D and O
    // (k for whole matrices, larger for tiles of bigger matrices)
    // desc: when given, chunk c is desc[c] = {first nonzero, end, slot of the piece
    // entering from the left or -1, slot of the piece leaving to the right, -1 when
    // nothing leaves, -2 when the whole chunk is one run that goes on} (a prepared
    // plan, see plan.cu) instead of the regular grid of `chunk` nonzeros.
    // storebit: a run whose segment value has this bit set overwrites its output
    // column instead of adding to it (0: always add).
    typedef Vec<S, VEC> V;
    typedef typename V::T VT;
    const int lane = threadIdx.x & (LPV - 1);
    const unsigned mask = worker_mask<LPV>();
    const long long c = ((long long)blockIdx.x * kThreads + threadIdx.x) / LPV;
    if (c >= nchunks) return;

    const int ktile = blockIdx.y * (LPV * NT * VEC);
    int eoff[NT];      // float offset of this lane's t-th element inside a column
    bool eok[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) {
        eoff[t] = ktile + (lane + t * LPV) * VEC;
        eok[t] = eoff[t] < k;
    }

    // [lo, hi) is the slice of the nonzero list this launch works on (the whole
    // list unless `range` points at two offsets); chunks are counted from lo.
    long long lo = 0, hi = nnz, j0, j1;
    long long hslot = c * 2, tslot = c * 2 + 1;
    int cur;
    bool head_open;
    int tail_code = 0;                 // plan: -1 nothing leaves to the right, else something does
    if (desc) {
        const int4 dc = __ldg(desc + c);
        j0 = dc.x; j1 = dc.y; hslot = dc.z; tslot = dc.w; tail_code = dc.w;
        cur = __ldg(seg + j0);
        head_open = dc.z >= 0;
    } else {
        lo = range ? (long long)__ldg(range) : 0;
        hi = range ? (long long)__ldg(range + 1) : nnz;
        j0 = lo + c * (long long)chunk;
        if (j0 >= hi) return;
        j1 = (j0 + chunk < hi) ? j0 + chunk : hi;
        cur = __ldg(seg + j0);
        head_open = (j0 > lo) && (__ldg(seg + j0 - 1) == cur);
    }

    VT acc[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t] = V::zero();

    auto flush = [&](bool tail_open) {
        if (!head_open && !tail_open) {
            S *o = O + (size_t)((unsigned)cur & segmask) * ld_o;
            const bool overwrite = ((unsigned)cur & storebit) != 0u;
#pragma unroll
            for (int t = 0; t < NT; t++)
                if (eok[t]) {
                    if (overwrite) {
                        V::st(o + eoff[t], acc[t]);
                    } else {
                        VT old = V::ld(o + eoff[t]);
                        V::add(old, acc[t]);
                        V::st(o + eoff[t], old);
                    }
                }
        } else {
            S *p = part + (size_t)(head_open ? hslot : tslot) * k;
#pragma unroll
            for (int t = 0; t < NT; t++)
                if (eok[t]) V::st(p + eoff[t], acc[t]);
        }
    };

    for (long long base = j0; base < j1; base += LPV) {
        long long jj = base + lane;
        if (jj >= j1) jj = j1 - 1;  // padded lanes repeat the last entry; never accumulated
        const int my_idx = __ldg(gidx + jj);
        const S my_val = __ldg(val + jj);
        const int my_seg = __ldg(seg + jj);
        const int cnt = (j1 - base < LPV) ? (int)(j1 - base) : LPV;
        for (int t0 = 0; t0 < cnt; t0 += U) {
            VT x[U][NT];
            int s[U];
            S v[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int src = (t0 + u) & (LPV - 1);
                const int i = __shfl_sync(mask, my_idx, src, LPV);
                v[u] = __shfl_sync(mask, my_val, src, LPV);
                s[u] = __shfl_sync(mask, my_seg, src, LPV);
                const S *d = D + (size_t)i * ld_d;
#pragma unroll
                for (int t = 0; t < NT; t++) x[u][t] = eok[t] ? V::ldg(d + eoff[t]) : V::zero();
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                if (t0 + u < cnt) {
                    if (s[u] != cur) {
                        flush(false);
                        cur = s[u];
                        head_open = false;
#pragma unroll
                        for (int t = 0; t < NT; t++) acc[t] = V::zero();
                    }
#pragma unroll
                    for (int t = 0; t < NT; t++) V::fma(acc[t], v[u], x[u][t]);
                }
            }
        }
    }
    const bool tail_open = desc ? (tail_code != -1) : ((j1 < hi) && (__ldg(seg + j1) == cur));
    flush(tail_open);
}

// One worker per chunk.  The worker whose chunk holds the START of a run that
// leaves the chunk to the right adds the stored pieces of the run in chunk
// order and adds the total to O.  Every other worker returns.
// Most runs that cross a boundary end in the very next chunk, so that case is
// one memory round trip: the piece leaving chunk c, the piece entering chunk
// c+1, the "does it go on" test and the current output column are independent
// loads issued together.  Longer runs (hot rows or long columns) continue
// four chunks per round trip.  The kernel is kept small in registers: it is
// latency bound and lives on occupancy.
template <typename S, int VEC, int LPV, int NT>
__global__ void __launch_bounds__(kThreads)
ga_fixup_kernel(int k, long long nnz, int chunk, long long nchunks,
                const int *__restrict__ seg, S *__restrict__ O,
                const S *__restrict__ part, const int *__restrict__ range, unsigned segmask, int ld_o) {
    typedef Vec<S, VEC> V;
    typedef typename V::T VT;
    const int lane = threadIdx.x & (LPV - 1);
    const long long c = ((long long)blockIdx.x * kThreads + threadIdx.x) / LPV;
    if (c >= nchunks) return;
    const long long lo = range ? (long long)__ldg(range) : 0;
    const long long hi = range ? (long long)__ldg(range + 1) : nnz;
    const long long j0 = lo + c * (long long)chunk;
    const long long j1 = j0 + chunk;
    if (j1 >= hi) return;
    const int s = __ldg(seg + j1 - 1);
    const int next = __ldg(seg + j1);
    const int prev = (j0 > lo) ? __ldg(seg + j0 - 1) : ~s;
    if (next != s) return;                                  // nothing leaves to the right
    if (prev == s) return;                                  // the run started further left

    const int ktile = blockIdx.y * (LPV * NT * VEC);
    const long long last = (hi - lo - 1) / chunk;           // index of the last chunk of the slice
    // does the run go on after chunk d (i.e. chunk d is all s and chunk d+1 starts with s)?
    // Both index loads are issued unconditionally (at a clamped, always valid position):
    // a short-circuit would make the second load wait for the first and serialise the walk.
    auto goes_on = [&](long long d) -> bool {
        const long long dc = d < last ? d : last - 1;        // last >= 1 here
        const long long dj1 = lo + (dc + 1) * (long long)chunk;
        const int a = __ldg(seg + dj1 - 1);
        const int b = __ldg(seg + dj1);
        return (d < last) & (a == s) & (b == s);
    };
    int eoff[NT];
    bool eok[NT];
    VT tot[NT], x1[NT], old[NT];
    S *o = O + (size_t)((unsigned)s & segmask) * ld_o;
#pragma unroll
    for (int t = 0; t < NT; t++) {
        eoff[t] = ktile + (lane + t * LPV) * VEC;
        eok[t] = eoff[t] < k;
        tot[t] = eok[t] ? V::ld(part + ((size_t)c * 2 + 1) * k + eoff[t]) : V::zero();
        x1[t] = eok[t] ? V::ld(part + ((size_t)(c + 1) * 2) * k + eoff[t]) : V::zero();
        old[t] = eok[t] ? V::ld(o + eoff[t]) : V::zero();
    }
    bool more = goes_on(c + 1);
#pragma unroll
    for (int t = 0; t < NT; t++) V::add(tot[t], x1[t]);

    constexpr int PF = 4;
    for (long long d = c + 2; more; d += PF) {
        VT x[PF][NT];
        bool g[PF];
#pragma unroll
        for (int q = 0; q < PF; q++) {
            const long long dd = (d + q <= last) ? d + q : last;
            const S *p = part + (size_t)dd * 2 * k;
#pragma unroll
            for (int t = 0; t < NT; t++) x[q][t] = eok[t] ? V::ld(p + eoff[t]) : V::zero();
            g[q] = goes_on(d + q);
        }
#pragma unroll
        for (int q = 0; q < PF; q++) {
            if (more) {
#pragma unroll
                for (int t = 0; t < NT; t++) V::add(tot[t], x[q][t]);
                more = g[q];
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NT; t++)
        if (eok[t]) {
            V::add(old[t], tot[t]);
            V::st(o + eoff[t], old[t]);
        }
}

// ---------------------------------------------------------------------------
// Fast paths for the common dense heights k = VEC*LPV*NT (fp32: 32, 64, 128, 256,
// 512; fp64: 16, 32, 64, 128, 256) with 16-byte aligned operands: every lane owns
// exactly NT 16-byte vectors (float4 / double2) of a column, so no bounds
// predicates are needed.
//
// The (index, value, segment) triples of the next LPV nonzeros are staged in
// shared memory with cp.async while the current LPV are processed, so the
// gathers never wait for an index load and the triple of nonzero t is one
// broadcast 16-byte shared load instead of three shuffles.  Gathers are issued
// U columns ahead of the FMAs that consume them (two register buffers), so a
// worker always has U..2U column loads in flight.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async4(void *smem_dst, const void *gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async8(void *smem_dst, const void *gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

template <int LPV> __device__ __forceinline__ void worker_sync(unsigned mask) {
    __syncwarp(mask);
}

// What the predicate-free kernels need to know about the scalar type: the 16-byte
// vector a lane loads, its arithmetic, and where the fields of a staged nonzero
// sit in its 16-byte shared-memory record.
//   float : {gather index, value bits, segment, source position}
//   double: {gather index, segment, value low word, value high word}
template <typename S> struct FastOps;
template <> struct FastOps<float> {
    typedef float4 vec;
    static constexpr int VEC = 4;
    static __device__ __forceinline__ vec zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
    static __device__ __forceinline__ void axpy(float v, const vec &x, vec &a) {
        a.x = fmaf(v, x.x, a.x); a.y = fmaf(v, x.y, a.y); a.z = fmaf(v, x.z, a.z); a.w = fmaf(v, x.w, a.w);
    }
    static __device__ __forceinline__ void add(vec &o, const vec &a) { o.x += a.x; o.y += a.y; o.z += a.z; o.w += a.w; }
    static __device__ __forceinline__ float dot(const vec &x, const vec &b, float s) {
        s = fmaf(x.x, b.x, s); s = fmaf(x.y, b.y, s); s = fmaf(x.z, b.z, s); s = fmaf(x.w, b.w, s);
        return s;
    }
    static __device__ __forceinline__ int seg(const int4 &m) { return m.z; }
    static __device__ __forceinline__ float val(const int4 &m) { return __int_as_float(m.y); }
    static __device__ __forceinline__ void stage_seg(int4 *dst, const int *src) { cp_async4(&dst->z, src); }
    static __device__ __forceinline__ void stage_val(int4 *dst, const float *src) { cp_async4(&dst->y, src); }
    static __device__ __forceinline__ int4 pad(int gidx, int sg) { return make_int4(gidx, 0, sg, -1); }   // value 0
};
template <> struct FastOps<double> {
    typedef double2 vec;
    static constexpr int VEC = 2;
    static __device__ __forceinline__ vec zero() { return make_double2(0.0, 0.0); }
    static __device__ __forceinline__ void axpy(double v, const vec &x, vec &a) { a.x = fma(v, x.x, a.x); a.y = fma(v, x.y, a.y); }
    static __device__ __forceinline__ void add(vec &o, const vec &a) { o.x += a.x; o.y += a.y; }
    static __device__ __forceinline__ double dot(const vec &x, const vec &b, double s) {
        s = fma(x.x, b.x, s); s = fma(x.y, b.y, s);
        return s;
    }
    static __device__ __forceinline__ int seg(const int4 &m) { return m.y; }
    static __device__ __forceinline__ double val(const int4 &m) { return __hiloint2double(m.w, m.z); }
    static __device__ __forceinline__ void stage_seg(int4 *dst, const int *src) { cp_async4(&dst->y, src); }
    static __device__ __forceinline__ void stage_val(int4 *dst, const double *src) { cp_async8(&dst->z, src); }
    static __device__ __forceinline__ int4 pad(int gidx, int sg) { return make_int4(gidx, sg, 0, 0); }    // value 0.0
};

template <typename S, int LPV, int NT, int U, int TPB, int MINB = 0>
__global__ void __launch_bounds__(TPB, MINB)
ga_chunk_fast_kernel(long long nnz, int chunk, long long nchunks,
                     const S *__restrict__ D, const S *__restrict__ val,
                     const int *__restrict__ gidx, const int *__restrict__ seg,
                     S *__restrict__ O, S *__restrict__ part,
                     const int *__restrict__ range, unsigned segmask) {
    typedef FastOps<S> F;
    typedef typename F::vec vec;
    constexpr int K = F::VEC * LPV * NT;   // dense height handled by this instantiation
    constexpr int WPB = TPB / LPV;         // workers per CTA
    constexpr int G = LPV / U;             // groups of U nonzeros per staged batch
    static_assert(LPV % U == 0, "U must divide LPV");
    __shared__ int4 meta[WPB][2][LPV];     // staged nonzeros, fields as FastOps<S> lays them out

    const int lane = threadIdx.x & (LPV - 1);
    const int w = threadIdx.x / LPV;
    const unsigned mask = worker_mask<LPV>();
    const long long c = (long long)blockIdx.x * WPB + w;
    if (c >= nchunks) return;

    const long long lo = range ? (long long)__ldg(range) : 0;
    const long long hi = range ? (long long)__ldg(range + 1) : nnz;
    const long long j0 = lo + c * (long long)chunk;
    if (j0 >= hi) return;
    const long long j1 = (j0 + chunk < hi) ? j0 + chunk : hi;
    const int nb = (int)((j1 - j0 + LPV - 1) / LPV);
    const S *Dl = D + lane * F::VEC;       // this lane's first 16-byte vector inside any column

    auto stage = [&](int buf, long long base) {
        const long long jj = base + lane;
        int4 *dst = &meta[w][buf][lane];
        if (jj < j1) {
            cp_async4(&dst->x, gidx + jj);
            F::stage_val(dst, val + jj);
            F::stage_seg(dst, seg + jj);
        } else {
            // padding of the last batch: repeat the last nonzero with value 0
            *dst = F::pad(__ldg(gidx + j1 - 1), __ldg(seg + j1 - 1));
        }
        cp_async_commit();
    };

    int cur = __ldg(seg + j0);
    const int seg_before = (j0 > lo) ? __ldg(seg + j0 - 1) : ~cur;
    const int seg_after = (j1 < hi) ? __ldg(seg + j1) : 0;      // fetched now, needed at the very end
    bool head_open = (j0 > lo) && (seg_before == cur);
    vec acc[NT];
    vec oldv[NT];      // current contents of the output column of the run, fetched when the run starts
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t] = F::zero();

    // The read half of the output's read-modify-write is issued at the start of a
    // run and only consumed when the run is flushed, so its latency overlaps the
    // gathers of the run.  Only this worker touches that column during the launch
    // (runs shared with a neighbour go to `part` instead), so the value cannot
    // change in between.
    auto prefetch_out = [&]() {
        const vec *o = reinterpret_cast<const vec *>(O + (size_t)((unsigned)cur & segmask) * K) + lane;
#pragma unroll
        for (int t = 0; t < NT; t++) oldv[t] = o[t * LPV];
    };

    auto flush = [&](bool tail_open) {
        if (!head_open && !tail_open) {
            vec *o = reinterpret_cast<vec *>(O + (size_t)((unsigned)cur & segmask) * K) + lane;
#pragma unroll
            for (int t = 0; t < NT; t++) {
                vec old = oldv[t];
                F::add(old, acc[t]);
                o[t * LPV] = old;
            }
        } else {
            vec *p = reinterpret_cast<vec *>(part + ((size_t)c * 2 + (head_open ? 0 : 1)) * K) + lane;
#pragma unroll
            for (int t = 0; t < NT; t++) p[t * LPV] = acc[t];
        }
    };

    stage(0, j0);
    prefetch_out();
    for (int b = 0; b < nb; b++) {
        if (b + 1 < nb) {
            stage((b + 1) & 1, j0 + (long long)(b + 1) * LPV);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        worker_sync<LPV>(mask);
        const int4 *mt = meta[w][b & 1];

        vec x[2][U][NT];
        int4 e[2][U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            e[0][u] = mt[u];
            const vec *d = reinterpret_cast<const vec *>(Dl + (size_t)e[0][u].x * K);
#pragma unroll
            for (int t = 0; t < NT; t++) x[0][u][t] = __ldg(d + t * LPV);
        }
#pragma unroll
        for (int g = 0; g < G; g++) {
            if (g + 1 < G) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    e[(g + 1) & 1][u] = mt[(g + 1) * U + u];
                    const vec *d = reinterpret_cast<const vec *>(Dl + (size_t)e[(g + 1) & 1][u].x * K);
#pragma unroll
                    for (int t = 0; t < NT; t++) x[(g + 1) & 1][u][t] = __ldg(d + t * LPV);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int4 m = e[g & 1][u];
                if (F::seg(m) != cur) {
                    flush(false);
                    cur = F::seg(m);
                    head_open = false;
                    prefetch_out();
#pragma unroll
                    for (int t = 0; t < NT; t++) acc[t] = F::zero();
                }
                const S v = F::val(m);
#pragma unroll
                for (int t = 0; t < NT; t++) F::axpy(v, x[g & 1][u][t], acc[t]);
            }
        }
        worker_sync<LPV>(mask);   // everyone is done with this buffer before it is staged again
    }
    const bool tail_open = (j1 < hi) && (seg_after == cur);
    flush(tail_open);
}

// Sampled dense-dense product, fast path (k = 32*NT 16-byte vectors, full warps).  The dot
// products of 8 consecutive nonzeros are reduced together: three exchange
// steps halve the number of live partials while doubling the lanes summed,
// then two plain xor steps finish, 9 shuffles per 8 nonzeros instead of 40.
// After four such groups lane l holds the result of nonzero (l&3)*8 + (l>>2)
// of the batch, and the 32 results go out as one 128-byte store.
template <typename S, int NT, int U, int TPB, bool ACCUM>
__global__ void __launch_bounds__(TPB)
dds_chunk_fast_kernel(long long nnz, int chunk, long long nchunks,
                      const S *__restrict__ A, const S *__restrict__ B,
                      const int *__restrict__ ir, const int *__restrict__ ic, S *__restrict__ P) {
    typedef FastOps<S> F;
    typedef typename F::vec vec;
    constexpr int LPV = 32;
    constexpr int K = F::VEC * LPV * NT;
    constexpr int WPB = TPB / LPV;
    static_assert(8 % U == 0, "U must divide 8");
    __shared__ int2 meta[WPB][2][LPV];     // {row, column}

    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    const unsigned mask = 0xffffffffu;
    const long long c = (long long)blockIdx.x * WPB + w;
    if (c >= nchunks) return;
    const long long j0 = c * (long long)chunk;
    const long long j1 = (j0 + chunk < nnz) ? j0 + chunk : nnz;
    const int nb = (int)((j1 - j0 + LPV - 1) / LPV);
    const S *Al = A + lane * F::VEC;
    const S *Bl = B + lane * F::VEC;

    auto stage = [&](int buf, long long base) {
        const long long jj = base + lane;
        int2 *dst = &meta[w][buf][lane];
        if (jj < j1) {
            cp_async4(&dst->x, ir + jj);
            cp_async4(&dst->y, ic + jj);
        } else {
            *dst = make_int2(__ldg(ir + j1 - 1), __ldg(ic + j1 - 1));
        }
        cp_async_commit();
    };

    int cur = -1;
    vec bv[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) bv[t] = F::zero();

    stage(0, j0);
    for (int b = 0; b < nb; b++) {
        const long long base = j0 + (long long)b * LPV;
        if (b + 1 < nb) {
            stage((b + 1) & 1, base + LPV);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp(mask);
        const int2 *mt = meta[w][b & 1];
        // my own result slot of this batch; start its read-modify-write early
        const int myslot = (lane & 3) * 8 + (lane >> 2);
        const long long myj = base + myslot;
        S old = 0;
        if (ACCUM && myj < j1) old = P[myj];
        S mine = 0;

        vec x[2][U][NT];
        int2 e[2][U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            e[0][u] = mt[u];
            const vec *a = reinterpret_cast<const vec *>(Al + (size_t)e[0][u].x * K);
#pragma unroll
            for (int t = 0; t < NT; t++) x[0][u][t] = __ldg(a + t * LPV);
        }
        S p[8];
#pragma unroll
        for (int g = 0; g < LPV / U; g++) {
            if (g + 1 < LPV / U) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    e[(g + 1) & 1][u] = mt[(g + 1) * U + u];
                    const vec *a = reinterpret_cast<const vec *>(Al + (size_t)e[(g + 1) & 1][u].x * K);
#pragma unroll
                    for (int t = 0; t < NT; t++) x[(g + 1) & 1][u][t] = __ldg(a + t * LPV);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int col = e[g & 1][u].y;
                if (col != cur) {
                    cur = col;
                    const vec *bp = reinterpret_cast<const vec *>(Bl + (size_t)cur * K);
#pragma unroll
                    for (int t = 0; t < NT; t++) bv[t] = __ldg(bp + t * LPV);
                }
                S s = 0;
#pragma unroll
                for (int t = 0; t < NT; t++) s = F::dot(x[g & 1][u][t], bv[t], s);
                p[(g * U + u) & 7] = s;        // position in the batch modulo 8 (compile-time: loops are unrolled)
            }
            if (((g * U + U - 1) & 7) == 7) {
                // reduce the 8 partial dot products p[0..7] of the last 8 nonzeros
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const S give = (lane & 16) ? p[i] : p[i + 4];
                    const S keep = (lane & 16) ? p[i + 4] : p[i];
                    p[i] = keep + __shfl_xor_sync(mask, give, 16);
                }
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const S give = (lane & 8) ? p[i] : p[i + 2];
                    const S keep = (lane & 8) ? p[i + 2] : p[i];
                    p[i] = keep + __shfl_xor_sync(mask, give, 8);
                }
                {
                    const S give = (lane & 4) ? p[0] : p[1];
                    const S keep = (lane & 4) ? p[1] : p[0];
                    p[0] = keep + __shfl_xor_sync(mask, give, 4);
                }
                p[0] += __shfl_xor_sync(mask, p[0], 2);
                p[0] += __shfl_xor_sync(mask, p[0], 1);
                // lane l now holds the dot product of nonzero (l >> 2) of this group of 8
                if ((lane & 3) == ((g * U + U - 1) >> 3)) mine = p[0];
            }
        }
        if (myj < j1) P[myj] = ACCUM ? old + mine : mine;
        __syncwarp(mask);
    }
}

// ---------------------------------------------------------------------------
// A*S and DDS(A,B,S) in one pass (k = 128 or 256 or 512, 16-byte aligned operands):
//     C[:, ic[j]] += val[j] * A[:, ir[j]]       and       P[j] += <A[:, ir[j]], B[:, ic[j]]>
// Both operations gather the same column of A for the same nonzero, and that gather
// (1 KB at k = 256, from L2 for most nonzeros) is what bounds either of them: done
// together it is paid once.  The kernel is ga_chunk_fast_kernel (runs of equal column,
// pieces of runs that cross a chunk boundary to `part`, ga_fixup_kernel afterwards)
// with the sampled product of dds_chunk_fast_kernel added on the gathered column: the
// column of B is reloaded when the run changes, eight dot products are reduced
// together, 32 results leave as one coalesced store.  No float atomics.
// ---------------------------------------------------------------------------
// Unlike ga_chunk_fast_kernel, the output column of a run is read when the run is flushed, not
// when it starts: columns of S are long runs, so that read is exposed once per ~100 nonzeros,
// and the registers it would occupy meanwhile are what lets five CTAs of this kernel share an
// SM (measured at k = 256: 9.6 ms against 12.9 ms with the early read and four CTAs).
template <int NT, int U, int TPB, int MINB>
__global__ void __launch_bounds__(TPB, MINB)
as_dds_chunk_fast_kernel(long long nnz, int chunk, long long nchunks,
                         const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ val,
                         const int *__restrict__ ir, const int *__restrict__ ic,
                         float *__restrict__ C, float *__restrict__ part, float *__restrict__ P) {
    constexpr int LPV = 32;
    constexpr int K = 4 * LPV * NT;
    constexpr int WPB = TPB / LPV;
    constexpr int G = LPV / U;
    static_assert(LPV % U == 0 && 8 % U == 0, "U must divide 8");
    __shared__ int4 meta[WPB][2][LPV];     // {row, value bits, column, unused}

    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    const unsigned mask = 0xffffffffu;
    const long long c = (long long)blockIdx.x * WPB + w;
    if (c >= nchunks) return;
    const long long j0 = c * (long long)chunk;
    if (j0 >= nnz) return;
    const long long j1 = (j0 + chunk < nnz) ? j0 + chunk : nnz;
    const int nb = (int)((j1 - j0 + LPV - 1) / LPV);
    const float *Al = A + lane * 4;
    const float *Bl = B + lane * 4;

    auto stage = [&](int buf, long long base) {
        const long long jj = base + lane;
        int4 *dst = &meta[w][buf][lane];
        if (jj < j1) {
            cp_async4(&dst->x, ir + jj);
            cp_async4(&dst->y, val + jj);
            cp_async4(&dst->z, ic + jj);
        } else {
            // padding of the last batch: repeat the last nonzero with value 0 (its dot product is dropped)
            *dst = make_int4(__ldg(ir + j1 - 1), 0, __ldg(ic + j1 - 1), 0);
        }
        cp_async_commit();
    };

    int cur = __ldg(ic + j0);
    const int seg_before = (j0 > 0) ? __ldg(ic + j0 - 1) : ~cur;
    const int seg_after = (j1 < nnz) ? __ldg(ic + j1) : 0;
    bool head_open = (j0 > 0) && (seg_before == cur);
    float4 acc[NT], bv[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t] = make_float4(0.f, 0.f, 0.f, 0.f);

    // at the start of a run: the column of B its dot products need
    auto start_run = [&]() {
        const float4 *bp = reinterpret_cast<const float4 *>(Bl + (size_t)cur * K);
#pragma unroll
        for (int t = 0; t < NT; t++) bv[t] = __ldg(bp + t * LPV);
    };
    auto flush = [&](bool tail_open) {
        if (!head_open && !tail_open) {
            float4 *o = reinterpret_cast<float4 *>(C + (size_t)cur * K) + lane;
#pragma unroll
            for (int t = 0; t < NT; t++) {
                float4 old = o[t * LPV];
                old.x += acc[t].x; old.y += acc[t].y; old.z += acc[t].z; old.w += acc[t].w;
                o[t * LPV] = old;
            }
        } else {
            float4 *p = reinterpret_cast<float4 *>(part + ((size_t)c * 2 + (head_open ? 0 : 1)) * K) + lane;
#pragma unroll
            for (int t = 0; t < NT; t++) p[t * LPV] = acc[t];
        }
    };

    stage(0, j0);
    start_run();
    for (int b = 0; b < nb; b++) {
        const long long base = j0 + (long long)b * LPV;
        if (b + 1 < nb) {
            stage((b + 1) & 1, base + LPV);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp(mask);
        const int4 *mt = meta[w][b & 1];
        // my own result slot of this batch; start its read-modify-write early
        const int myslot = (lane & 3) * 8 + (lane >> 2);
        const long long myj = base + myslot;
        float old = 0.f;
        if (myj < j1) old = P[myj];
        float mine = 0.f;

        float4 x[2][U][NT];
        int4 e[2][U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            e[0][u] = mt[u];
            const float4 *a = reinterpret_cast<const float4 *>(Al + (size_t)e[0][u].x * K);
#pragma unroll
            for (int t = 0; t < NT; t++) x[0][u][t] = __ldg(a + t * LPV);
        }
        float p[8];
#pragma unroll
        for (int g = 0; g < G; g++) {
            if (g + 1 < G) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    e[(g + 1) & 1][u] = mt[(g + 1) * U + u];
                    const float4 *a = reinterpret_cast<const float4 *>(Al + (size_t)e[(g + 1) & 1][u].x * K);
#pragma unroll
                    for (int t = 0; t < NT; t++) x[(g + 1) & 1][u][t] = __ldg(a + t * LPV);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int4 m = e[g & 1][u];
                if (m.z != cur) {
                    flush(false);
                    cur = m.z;
                    head_open = false;
                    start_run();
#pragma unroll
                    for (int t = 0; t < NT; t++) acc[t] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                const float v = __int_as_float(m.y);
                float s = 0.f;
#pragma unroll
                for (int t = 0; t < NT; t++) {
                    const float4 xv = x[g & 1][u][t];
                    acc[t].x = fmaf(v, xv.x, acc[t].x); acc[t].y = fmaf(v, xv.y, acc[t].y);
                    acc[t].z = fmaf(v, xv.z, acc[t].z); acc[t].w = fmaf(v, xv.w, acc[t].w);
                    s = fmaf(xv.x, bv[t].x, s); s = fmaf(xv.y, bv[t].y, s);
                    s = fmaf(xv.z, bv[t].z, s); s = fmaf(xv.w, bv[t].w, s);
                }
                const int pos = g * U + u;             // position in the batch (compile-time: loops are unrolled)
                p[pos & 7] = s;
                if ((pos & 7) == 7) {
                    // reduce the 8 partial dot products of nonzeros pos-7 .. pos
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float give = (lane & 16) ? p[i] : p[i + 4];
                        const float keep = (lane & 16) ? p[i + 4] : p[i];
                        p[i] = keep + __shfl_xor_sync(mask, give, 16);
                    }
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const float give = (lane & 8) ? p[i] : p[i + 2];
                        const float keep = (lane & 8) ? p[i + 2] : p[i];
                        p[i] = keep + __shfl_xor_sync(mask, give, 8);
                    }
                    {
                        const float give = (lane & 4) ? p[0] : p[1];
                        const float keep = (lane & 4) ? p[1] : p[0];
                        p[0] = keep + __shfl_xor_sync(mask, give, 4);
                    }
                    p[0] += __shfl_xor_sync(mask, p[0], 2);
                    p[0] += __shfl_xor_sync(mask, p[0], 1);
                    // lane l now holds the dot product of nonzero (l >> 2) of this group of 8
                    if ((lane & 3) == (pos >> 3)) mine = p[0];
                }
            }
        }
        if (myj < j1) P[myj] = old + mine;
        __syncwarp(mask);
    }
    const bool tail_open = (j1 < nnz) && (seg_after == cur);
    flush(tail_open);
}

// ---------------------------------------------------------------------------
// Sampled dense-dense product:  P[j] (+)= <A[:, ir[j]], B[:, ic[j]]>
//
// One worker per chunk of nonzeros.  The B column is kept in registers while
// the column index stays the same (ic is non-decreasing, so it is re-read
// about once per column); A columns are gathered U at a time with 16-byte
// loads; the dot product is finished with xor-shuffles inside the worker; the
// LPV results of one batch are written back as one coalesced store.
// A k-tile wider than LPV*NT*VEC is handled by looping over tiles inside the
// worker so that P is written once.
// ---------------------------------------------------------------------------
template <typename S, int VEC, int LPV, int NT, int U, bool ACCUM>
__global__ void __launch_bounds__(kThreads)
dds_chunk_kernel(int k, long long nnz, int chunk, long long nchunks,
                 const S *__restrict__ A, const S *__restrict__ B,
                 const int *__restrict__ ir, const int *__restrict__ ic, S *__restrict__ P) {
    typedef Vec<S, VEC> V;
    typedef typename V::T VT;
    const int lane = threadIdx.x & (LPV - 1);
    const unsigned mask = worker_mask<LPV>();
    const long long c = ((long long)blockIdx.x * kThreads + threadIdx.x) / LPV;
    if (c >= nchunks) return;
    constexpr int TILE = LPV * NT * VEC;
    const int ntiles = (k + TILE - 1) / TILE;

    const long long j0 = c * (long long)chunk;
    const long long j1 = (j0 + chunk < nnz) ? j0 + chunk : nnz;

    int cur = -1;  // column whose B vector is held in b[]
    VT b[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) b[t] = V::zero();

    for (long long base = j0; base < j1; base += LPV) {
        long long jj = base + lane;
        const bool mine_ok = jj < j1;
        if (!mine_ok) jj = j1 - 1;
        const int my_ir = __ldg(ir + jj);
        const int my_ic = __ldg(ic + jj);
        const int cnt = (j1 - base < LPV) ? (int)(j1 - base) : LPV;
        S mine = 0;
        for (int tile = 0; tile < ntiles; tile++) {
            int eoff[NT];
            bool eok[NT];
#pragma unroll
            for (int t = 0; t < NT; t++) {
                eoff[t] = tile * TILE + (lane + t * LPV) * VEC;
                eok[t] = eoff[t] < k;
            }
            if (ntiles > 1) cur = -1;  // b[] belongs to another tile
            for (int t0 = 0; t0 < cnt; t0 += U) {
                VT x[U][NT];
                int cc[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int src = (t0 + u) & (LPV - 1);
                    const int i = __shfl_sync(mask, my_ir, src, LPV);
                    cc[u] = __shfl_sync(mask, my_ic, src, LPV);
                    const S *a = A + (size_t)i * k;
#pragma unroll
                    for (int t = 0; t < NT; t++) x[u][t] = eok[t] ? V::ldg(a + eoff[t]) : V::zero();
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
                    if (t0 + u < cnt) {
                        if (cc[u] != cur) {
                            cur = cc[u];
                            const S *bp = B + (size_t)cur * k;
#pragma unroll
                            for (int t = 0; t < NT; t++) b[t] = eok[t] ? V::ldg(bp + eoff[t]) : V::zero();
                        }
                        S p = 0;
#pragma unroll
                        for (int t = 0; t < NT; t++) p = V::dot(x[u][t], b[t], p);
#pragma unroll
                        for (int off = LPV / 2; off > 0; off >>= 1) p += __shfl_xor_sync(mask, p, off, LPV);
                        if (lane == t0 + u) mine += p;
                    }
                }
            }
        }
        if (mine_ok) {
            if (ACCUM) P[jj] = P[jj] + mine;
            else P[jj] = mine;
        }
    }
}

}  // namespace bidmat
