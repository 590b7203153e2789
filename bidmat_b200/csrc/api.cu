// Host side of the C ABI declared in include/bidmat_b200.h: argument checks,
// kernel selection by the dense height k, the per-device scratch workspace and
// the row-sort that turns the CSC nonzero list into the row-major order B*^S
// needs.  Built for sm_100a only.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>
#include <vector>

#include "../../include/bidmat_b200.h"
#include "auto_plan.cuh"
#include "launchers.cuh"
#include "structure_kernels.cuh"
#include "edgeops.cuh"
#include "tile_compact.cuh"

using namespace bidmat;

namespace {


template <typename S>
int dsmult_impl(int nrows, int ncols, int nnz, const S *A, const S *Bdata,
                             const int *Bir, const int *Bic, S *C, cudaStream_t st_in) {
    if (nrows < 0 || ncols < 0 || nnz < 0) return (int)cudaErrorInvalidValue;
    if (nnz == 0 || nrows == 0) return 0;
    if (!A || !Bdata || !Bir || !Bic || !C) return (int)cudaErrorInvalidValue;
    cudaStream_t st = st_in;
    const Shape s = pick_shape(nrows, is16(A) && is16(C), 16 / (int)sizeof(S));
    const int chunk = pick_chunk(nnz, s.lpv);
    WorkspaceLease ws(pad256(ga_part_floats(nrows, nnz, chunk) * sizeof(S)) + 256, st);
    if (ws.err != cudaSuccess) return (int)ws.err;
    S *part = ws.take<S>(ga_part_floats(nrows, nnz, chunk));
    return (int)launch_ga<S>(nrows, nnz, A, Bdata, Bir, Bic, C, part, chunk, s, st, "dsmult_ga_chunk");
}

template <typename S>
int dsmultT_impl(int nrows, int ncols, int nnz, const S *A, const S *Bdata,
                              const int *Bir, const int *Bic, S *C, int m_hint,
                              cudaStream_t st_in) {
    if (nrows < 0 || ncols < 0 || nnz < 0) return (int)cudaErrorInvalidValue;
    if (nnz == 0 || nrows == 0) return 0;
    if (!A || !Bdata || !Bir || !Bic || !C) return (int)cudaErrorInvalidValue;
    cudaStream_t st = st_in;
    const size_t n = (size_t)nnz;
    const Shape s = pick_shape(nrows, is16(A) && is16(C), 16 / (int)sizeof(S));

    const int ntiles = (int)((n + kSortTile - 1) / kSortTile);
    size_t need = 4 * pad256(n * 4) + 2 * pad256(n * sizeof(S)) + pad256((size_t)256 * ntiles * 4) + 4 * pad256(4096) + pad256(256 * kSortScanSegs * 4) + 4096;
    // Partial-sum scratch: enough chunk slots for the whole list or for any single
    // column block, whichever chunk length pick_chunk gives them.
    const int chunk_all = pick_chunk(nnz, s.lpv);
    const long long cap_chunks = max_chunks_for(nnz, s.lpv);
    const size_t part_floats = (size_t)cap_chunks * 2 * (size_t)nrows;
    need += pad256(part_floats * sizeof(S));
    WorkspaceLease ws(need, st);
    if (ws.err != cudaSuccess) return (int)ws.err;
    unsigned *keys[2] = {ws.take<unsigned>(n), ws.take<unsigned>(n)};
    int *cols[2] = {ws.take<int>(n), ws.take<int>(n)};
    S *vals[2] = {ws.take<S>(n), ws.take<S>(n)};
    int *counts = ws.take<int>((size_t)256 * ntiles);
    int *totals = ws.take<int>(256 * kSortScanSegs);   // per (digit, scan segment)
    int *maxrow = ws.take<int>(1);
    int *offsets = ws.take<int>(1024);
    S *part = ws.take<S>(part_floats);

    cudaError_t err;
    int rowbits;
    if (m_hint > 0) {
        rowbits = ceil_log2((unsigned long long)m_hint);
    } else {
        err = cudaMemsetAsync(maxrow, 0, sizeof(int), st);
        if (err != cudaSuccess) return (int)err;
        max_int_kernel<<<148 * 8, 256, 0, st>>>(nnz, Bir, maxrow);
        g_launches += 1;
        int h = 0;
        err = cudaMemcpyAsync(&h, maxrow, sizeof(int), cudaMemcpyDeviceToHost, st);
        if (err == cudaSuccess) err = cudaStreamSynchronize(st);
        if (err != cudaSuccess) return (int)err;
        if (h < 0) return (int)cudaErrorInvalidValue;
        rowbits = ceil_log2((unsigned long long)h + 1);
    }
    BlockLayout lay;
    if (!choose_block_layout(nrows, ncols, nnz, sizeof(S), rowbits, m_hint > 0 ? (double)m_hint : 0.0, 32, &lay))
        return (int)cudaErrorInvalidValue;
    const int nblocks = lay.nblocks, passes = lay.passes;
    rowbits = lay.rowbits;
    const SortKeySpec ks{lay.colshift, lay.rowbits};
    const unsigned rowmask = lay.rowmask;

    const int cur = run_rowsort<S>(nnz, passes, ks, Bir, Bic, Bdata, keys, cols, vals, nullptr, nullptr, nullptr, counts,
                                totals, st);
    err = cudaGetLastError();
    if (err != cudaSuccess) return (int)err;
    const int *seg = reinterpret_cast<const int *>(keys[cur]);

    if (nblocks == 1) {
        return (int)launch_ga<S>(nrows, nnz, A, vals[cur], cols[cur], seg, C, part, chunk_all, s, st, "dsmultT_ga_chunk",
                              nnz, nullptr, rowmask);
    }
    // slice boundaries of the column blocks in the sorted list
    block_offsets_kernel<<<(nblocks + 256) / 256, 256, 0, st>>>(nnz, nblocks, rowbits, keys[cur], offsets);
    g_launches += 1;
    std::vector<int> h_off((size_t)nblocks + 1);
    err = cudaMemcpyAsync(h_off.data(), offsets, sizeof(int) * (nblocks + 1), cudaMemcpyDeviceToHost, st);
    if (err == cudaSuccess) err = cudaStreamSynchronize(st);
    if (err != cudaSuccess) return (int)err;
    for (int b = 0; b < nblocks; b++) {
        const long long count = (long long)h_off[b + 1] - h_off[b];
        if (count <= 0) continue;
        int chunk = pick_chunk(count, s.lpv);
        if (ga_part_floats(nrows, count, chunk) > part_floats) chunk = chunk_all;
        err = launch_ga<S>(nrows, nnz, A, vals[cur], cols[cur], seg, C, part, chunk, s, st, "dsmultT_ga_chunk", count,
                        offsets + b, rowmask);
        if (err != cudaSuccess) return (int)err;
    }
    return 0;
}

template <typename S>
int dds_impl(int nrows, int nnz, const S *A, const S *B, const int *Cir,
                          const int *Cic, S *P, cudaStream_t st_in) {
    if (nrows < 0 || nnz < 0) return (int)cudaErrorInvalidValue;
    if (nnz == 0) return 0;
    if (!A || !B || !Cir || !Cic || !P) return (int)cudaErrorInvalidValue;
    if (nrows == 0) return 0;
    return (int)launch_dds<S, true>(nrows, nnz, A, B, Cir, Cic, P, st_in);
}

template <typename S>
int dds0_impl(int nrows, int ncols, int nnz, const S *A, const S *B,
                           const int *Cir, const int *Cjc, S *P, cudaStream_t st_in) {
    if (nrows < 0 || ncols < 0 || nnz < 0) return (int)cudaErrorInvalidValue;
    if (nnz == 0 || ncols == 0) return 0;
    if (!A || !B || !Cir || !Cjc || !P) return (int)cudaErrorInvalidValue;
    cudaStream_t st = st_in;
    if (nrows == 0) return (int)cudaMemsetAsync(P, 0, (size_t)nnz * sizeof(S), st);
    WorkspaceLease ws(pad256((size_t)nnz * 4) + 256, st);
    if (ws.err != cudaSuccess) return (int)ws.err;
    int *ic = ws.take<int>((size_t)nnz);
    expand_jc_kernel<<<(unsigned)(((size_t)nnz + kThreads - 1) / kThreads), kThreads, 0, st>>>(ncols, nnz, Cjc, ic);
    g_launches += 1;
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return (int)err;
    return (int)launch_dds<S, false>(nrows, nnz, A, B, Cir, ic, P, st);
}

template <typename S>
int sdop_common(int nnz, S *A, const int *idx, const S *B, int len, int opn) {
    if (nnz < 0 || len < 0 || opn < 0 || opn >= kNumBinops) return (int)cudaErrorInvalidValue;
    if (nnz == 0) return 0;
    if (!A || !B || (len > 1 && !idx)) return (int)cudaErrorInvalidValue;
    cudaStream_t st = cudaStreamPerThread;
    size_t blocks = ((size_t)nnz + kThreads - 1) / kThreads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    sdop_kernel<S><<<(unsigned)blocks, kThreads, 0, st>>>(nnz, A, len > 1 ? idx : nullptr, B, opn);
    g_launches += 1;
    return finish_sync(cudaGetLastError(), st);
}

// B[seg[j]] += P[j] for a non-decreasing seg: segmented sum, then the fix-up of the runs
// that cross chunk boundaries (the gather-accumulate fix-up with one element per column).
template <typename S>
cudaError_t launch_segsum(long long nnz, const S *P, const int *seg, S *B, S *part, cudaStream_t st) {
    constexpr int ITEMS = 16;
    constexpr int CHUNK = 32 * ITEMS;
    const long long nchunks = (nnz + CHUNK - 1) / CHUNK;
    {
        ScopedSpan sp("spsum_segsum", st);
        segsum_chunk_kernel<S, ITEMS><<<blocks_for(nchunks, 32), kThreads, 0, st>>>(nnz, nchunks, P, seg, B, part);
    }
    if (nchunks > 1)
        ga_fixup_kernel<S, 1, 8, 1><<<blocks_for(nchunks, 8), kThreads, 0, st>>>(1, nnz, CHUNK, nchunks, seg, B, part,
                                                                                 nullptr, 0xffffffffu, 1);
    g_launches += (nchunks > 1) ? 2 : 1;
    return cudaGetLastError();
}

template <typename S>
int spsum_impl(int nrows, int ncols, int nnz, const int *Air, const int *Aic, const S *P, S *B, int n) {
    if (nrows < 0 || ncols < 0 || nnz < 0) return (int)cudaErrorInvalidValue;
    if (nnz == 0) return 0;
    if (!Air || !Aic || !P || !B) return (int)cudaErrorInvalidValue;
    cudaStream_t st = cudaStreamPerThread;
    const size_t n_ = (size_t)nnz;
    const size_t part_elems = 2 * ((n_ + 511) / 512) + 2;
    if (n == 1) {
        // B(1 x ncols)[ic[j]] += P[j]: the column indices are already sorted
        WorkspaceLease ws(pad256(part_elems * sizeof(S)) + 256, st);
        if (ws.err != cudaSuccess) return (int)ws.err;
        S *part = ws.take<S>(part_elems);
        return finish_sync(launch_segsum<S>(nnz, P, Aic, B, part, st), st);
    }
    // B(nrows x 1)[ir[j]] += P[j]: stable sort of (row, value) by row first, then the same kernel
    const int ntiles = (int)((n_ + kSortTile - 1) / kSortTile);
    int rowbits = ceil_log2((unsigned long long)(nrows > 0 ? nrows : 1));
    if (rowbits < 1) rowbits = 1;
    if (rowbits > 31) return (int)cudaErrorInvalidValue;
    WorkspaceLease ws(2 * pad256(n_ * 4) + 2 * pad256(n_ * sizeof(S)) + pad256((size_t)256 * ntiles * 4) +
                          pad256(256 * kSortScanSegs * 4) + pad256(part_elems * sizeof(S)) + 4096, st);
    if (ws.err != cudaSuccess) return (int)ws.err;
    unsigned *keys[2] = {ws.take<unsigned>(n_), ws.take<unsigned>(n_)};
    int *cols[2] = {nullptr, nullptr};          // the sums need no columns: (row, value) pairs are sorted
    S *vals[2] = {ws.take<S>(n_), ws.take<S>(n_)};
    int *counts = ws.take<int>((size_t)256 * ntiles);
    int *totals = ws.take<int>(256 * kSortScanSegs);
    S *part = ws.take<S>(part_elems);
    const int cur = run_rowsort<S>(nnz, (rowbits + 7) / 8, SortKeySpec{31, rowbits}, Air, nullptr, P, keys, cols, vals,
                                   nullptr, nullptr, nullptr, counts, totals, st);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return (int)err;
    return finish_sync(launch_segsum<S>(nnz, vals[cur], reinterpret_cast<const int *>(keys[cur]), B, part, st), st);
}

}  // namespace

extern "C" {

int bidmat_b200_dsmult_async(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                             const int *Bir, const int *Bic, float *C, bidmat_stream_t stream) {
    return dsmult_impl<float>(nrows, ncols, nnz, A, Bdata, Bir, Bic, C, as_stream(stream));
}

int bidmat_b200_dsmultT_async(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                              const int *Bir, const int *Bic, float *C, int m_hint,
                              bidmat_stream_t stream) {
    return dsmultT_impl<float>(nrows, ncols, nnz, A, Bdata, Bir, Bic, C, m_hint, as_stream(stream));
}

int bidmat_b200_dds_async(int nrows, int nnz, const float *A, const float *B, const int *Cir,
                          const int *Cic, float *P, bidmat_stream_t stream) {
    return dds_impl<float>(nrows, nnz, A, B, Cir, Cic, P, as_stream(stream));
}

int bidmat_b200_dsmult_dds_async(int nrows, int ncols, int nnz, const float *A, const float *B, const float *Sdata,
                                 const int *Sir, const int *Sic, float *C, float *P, bidmat_stream_t stream) {
    if (nrows < 0 || ncols < 0 || nnz < 0) return (int)cudaErrorInvalidValue;
    if (nnz == 0 || nrows == 0) return 0;
    if (!A || !B || !Sdata || !Sir || !Sic || !C || !P) return (int)cudaErrorInvalidValue;
    cudaStream_t st = as_stream(stream);
    {
        const int chunk = pick_chunk(nnz, 32);
        WorkspaceLease ws(pad256(ga_part_floats(nrows, nnz, chunk) * sizeof(float)) + 256, st);
        if (ws.err != cudaSuccess) return (int)ws.err;
        float *part = ws.take<float>(ga_part_floats(nrows, nnz, chunk));
        cudaError_t err = cudaSuccess;
        if (launch_as_dds(nrows, nnz, A, B, Sdata, Sir, Sic, C, P, part, chunk, st, &err)) return (int)err;
    }
    // shapes the fused kernel does not cover: the two operations one after the other
    const int e = dsmult_impl<float>(nrows, ncols, nnz, A, Sdata, Sir, Sic, C, st);
    if (e != 0) return e;
    return dds_impl<float>(nrows, nnz, A, B, Sir, Sic, P, st);
}

int bidmat_b200_dds0_async(int nrows, int ncols, int nnz, const float *A, const float *B,
                           const int *Cir, const int *Cjc, float *P, bidmat_stream_t stream) {
    return dds0_impl<float>(nrows, ncols, nnz, A, B, Cir, Cjc, P, as_stream(stream));
}

int bidmat_b200_transpose_csc(int nrows, int ncols, int nnz, const int *ir, const int *ic, const float *data,
                              int *t_ir, int *t_ic, int *t_jc, float *t_data, bidmat_stream_t stream) {
    if (nrows < 0 || ncols < 0 || nnz < 0) return (int)cudaErrorInvalidValue;
    cudaStream_t st = as_stream(stream);
    if (nnz == 0) {
        if (t_jc) return (int)cudaMemsetAsync(t_jc, 0, ((size_t)nrows + 1) * sizeof(int), st);
        return 0;
    }
    if (!ir || !ic || !data || !t_ir || !t_ic || !t_data || nrows == 0) return (int)cudaErrorInvalidValue;
    const size_t n = (size_t)nnz;
    const int ntiles = (int)((n + kSortTile - 1) / kSortTile);
    int rowbits = ceil_log2((unsigned long long)nrows);
    if (rowbits < 1) rowbits = 1;
    if (rowbits > 31) return (int)cudaErrorInvalidValue;
    const int passes = (rowbits + 7) / 8;
    WorkspaceLease ws(6 * pad256(n * 4) + pad256((size_t)256 * ntiles * 4) + pad256(256 * kSortScanSegs * 4) + 4096, st);
    if (ws.err != cudaSuccess) return (int)ws.err;
    unsigned *keys[2] = {ws.take<unsigned>(n), ws.take<unsigned>(n)};
    int *cols[2] = {ws.take<int>(n), ws.take<int>(n)};
    float *vals[2] = {ws.take<float>(n), ws.take<float>(n)};
    int *counts = ws.take<int>((size_t)256 * ntiles);
    int *totals = ws.take<int>(256 * kSortScanSegs);
    // key = old row (the new column); payload = (old column = new row, value).  The
    // sort is stable and ic is non-decreasing, so the new rows come out ascending
    // inside every new column, as a CSC matrix needs.
    run_rowsort<float>(nnz, passes, SortKeySpec{31, rowbits}, ir, ic, data, keys, cols, vals,
                reinterpret_cast<unsigned *>(t_ic), t_ir, t_data, counts, totals, st);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return (int)err;
    if (t_jc) {
        compress_ic_kernel<<<(unsigned)((n + kThreads - 1) / kThreads), kThreads, 0, st>>>(nrows, nnz, t_ic, t_jc);
        g_launches += 1;
        err = cudaGetLastError();
    }
    return (int)err;
}

int bidmat_b200_dsmult(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                       const int *Bir, const int *Bic, float *C) {
    if (nrows >= 0 && ncols >= 0 && (nnz == 0 || nrows == 0)) return 0;  // nothing to do, nothing to wait for
    int e = bidmat_b200_dsmult_async(nrows, ncols, nnz, A, Bdata, Bir, Bic, C, cudaStreamPerThread);
    return finish_sync((cudaError_t)e, cudaStreamPerThread);
}

int bidmat_b200_dsmultT(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                        const int *Bir, const int *Bic, float *C) {
    if (nrows >= 0 && ncols >= 0 && (nnz == 0 || nrows == 0)) return 0;
    // a structure the library keeps a plan for (bidmat_b200_set_auto_plan) skips the sort
    int handled = 0, m_seen = 0;
    int e = auto_plan_dsmultT(4, nrows, ncols, nnz, A, Bdata, Bir, Bic, C, &handled, &m_seen);
    if (handled || e != 0) return e;
    e = bidmat_b200_dsmultT_async(nrows, ncols, nnz, A, Bdata, Bir, Bic, C, m_seen, cudaStreamPerThread);
    return finish_sync((cudaError_t)e, cudaStreamPerThread);
}

int bidmat_b200_dds(int nrows, int nnz, const float *A, const float *B, const int *Cir,
                    const int *Cic, float *P) {
    if (nrows >= 0 && nnz == 0) return 0;
    int e = bidmat_b200_dds_async(nrows, nnz, A, B, Cir, Cic, P, cudaStreamPerThread);
    return finish_sync((cudaError_t)e, cudaStreamPerThread);
}

int bidmat_b200_dds0(int nrows, int ncols, const float *A, const float *B, const int *Cir,
                     const int *Cjc, float *P) {
    if (nrows < 0 || ncols < 0) return (int)cudaErrorInvalidValue;
    if (ncols == 0) return 0;
    if (!Cjc) return (int)cudaErrorInvalidValue;
    // nnz is not part of the reference signature: it is the last column pointer.
    int nnz = 0;
    cudaError_t err = cudaMemcpyAsync(&nnz, Cjc + ncols, sizeof(int), cudaMemcpyDeviceToHost, cudaStreamPerThread);
    if (err == cudaSuccess) err = cudaStreamSynchronize(cudaStreamPerThread);
    if (err != cudaSuccess) return (int)err;
    int e = bidmat_b200_dds0_async(nrows, ncols, nnz, A, B, Cir, Cjc, P, cudaStreamPerThread);
    return finish_sync((cudaError_t)e, cudaStreamPerThread);
}

// ---- double-precision twins (BIDMat's CUMATD natives)
int bidmat_b200_dsmult_f64_async(int nrows, int ncols, int nnz, const double *A, const double *Bdata,
                                 const int *Bir, const int *Bic, double *C, bidmat_stream_t stream) {
    return dsmult_impl<double>(nrows, ncols, nnz, A, Bdata, Bir, Bic, C, as_stream(stream));
}

int bidmat_b200_dsmultT_f64_async(int nrows, int ncols, int nnz, const double *A, const double *Bdata,
                                  const int *Bir, const int *Bic, double *C, int m_hint, bidmat_stream_t stream) {
    return dsmultT_impl<double>(nrows, ncols, nnz, A, Bdata, Bir, Bic, C, m_hint, as_stream(stream));
}

int bidmat_b200_dds_f64_async(int nrows, int nnz, const double *A, const double *B, const int *Cir,
                              const int *Cic, double *P, bidmat_stream_t stream) {
    return dds_impl<double>(nrows, nnz, A, B, Cir, Cic, P, as_stream(stream));
}

int bidmat_b200_dsmult_f64(int nrows, int ncols, int nnz, const double *A, const double *Bdata,
                           const int *Bir, const int *Bic, double *C) {
    if (nrows >= 0 && ncols >= 0 && (nnz == 0 || nrows == 0)) return 0;
    int e = dsmult_impl<double>(nrows, ncols, nnz, A, Bdata, Bir, Bic, C, cudaStreamPerThread);
    return finish_sync((cudaError_t)e, cudaStreamPerThread);
}

int bidmat_b200_dsmultT_f64(int nrows, int ncols, int nnz, const double *A, const double *Bdata,
                            const int *Bir, const int *Bic, double *C) {
    if (nrows >= 0 && ncols >= 0 && (nnz == 0 || nrows == 0)) return 0;
    int handled = 0, m_seen = 0;
    int e = auto_plan_dsmultT(8, nrows, ncols, nnz, A, Bdata, Bir, Bic, C, &handled, &m_seen);
    if (handled || e != 0) return e;
    e = dsmultT_impl<double>(nrows, ncols, nnz, A, Bdata, Bir, Bic, C, m_seen, cudaStreamPerThread);
    return finish_sync((cudaError_t)e, cudaStreamPerThread);
}

int bidmat_b200_dds_f64(int nrows, int nnz, const double *A, const double *B, const int *Cir,
                        const int *Cic, double *P) {
    if (nrows >= 0 && nnz == 0) return 0;
    int e = dds_impl<double>(nrows, nnz, A, B, Cir, Cic, P, cudaStreamPerThread);
    return finish_sync((cudaError_t)e, cudaStreamPerThread);
}

int bidmat_b200_dds0_f64(int nrows, int ncols, const double *A, const double *B, const int *Cir,
                         const int *Cjc, double *P) {
    if (nrows < 0 || ncols < 0) return (int)cudaErrorInvalidValue;
    if (ncols == 0) return 0;
    if (!Cjc) return (int)cudaErrorInvalidValue;
    int nnz = 0;
    cudaError_t err = cudaMemcpyAsync(&nnz, Cjc + ncols, sizeof(int), cudaMemcpyDeviceToHost, cudaStreamPerThread);
    if (err == cudaSuccess) err = cudaStreamSynchronize(cudaStreamPerThread);
    if (err != cudaSuccess) return (int)err;
    int e = dds0_impl<double>(nrows, ncols, nnz, A, B, Cir, Cjc, P, cudaStreamPerThread);
    return finish_sync((cudaError_t)e, cudaStreamPerThread);
}

int bidmat_b200_dsmult_tune(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                            const int *Bir, const int *Bic, float *C, int, int) {
    return bidmat_b200_dsmult(nrows, ncols, nnz, A, Bdata, Bir, Bic, C);
}

int bidmat_b200_dsmultx_tune(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                             const int *Bir, const int *Bic, float *C, int, int, int) {
    return bidmat_b200_dsmult(nrows, ncols, nnz, A, Bdata, Bir, Bic, C);
}

int bidmat_b200_expand_jc(int ncols, int nnz, const int *jc, int *ic, bidmat_stream_t stream) {
    if (ncols < 0 || nnz < 0) return (int)cudaErrorInvalidValue;
    if (nnz == 0) return 0;
    if (!jc || !ic || ncols == 0) return (int)cudaErrorInvalidValue;
    expand_jc_kernel<<<(unsigned)(((size_t)nnz + kThreads - 1) / kThreads), kThreads, 0, as_stream(stream)>>>(ncols, nnz, jc, ic);
    g_launches += 1;
    return (int)cudaGetLastError();
}

int bidmat_b200_compress_ic(int ncols, int nnz, const int *ic, int *jc, bidmat_stream_t stream) {
    if (ncols < 0 || nnz < 0) return (int)cudaErrorInvalidValue;
    if (!jc || (nnz > 0 && !ic)) return (int)cudaErrorInvalidValue;
    const size_t threads = nnz > 0 ? (size_t)nnz : (size_t)ncols + 1;
    compress_ic_kernel<<<(unsigned)((threads + kThreads - 1) / kThreads), kThreads, 0, as_stream(stream)>>>(ncols, nnz, ic, jc);
    g_launches += 1;
    return (int)cudaGetLastError();
}

int bidmat_b200_check_structure(int m, int ncols, int nnz, const int *ir, const int *ic) {
    if (m < 0 || ncols < 0 || nnz < 0) return (int)cudaErrorInvalidValue;
    if (nnz == 0) return 0;
    if (!ir || !ic) return (int)cudaErrorInvalidValue;
    cudaStream_t st = cudaStreamPerThread;
    WorkspaceLease ws(512, st);
    if (ws.err != cudaSuccess) return (int)ws.err;
    int *flags = ws.take<int>(1);
    cudaError_t err = cudaMemsetAsync(flags, 0, sizeof(int), st);
    if (err != cudaSuccess) return (int)err;
    check_structure_kernel<<<(unsigned)(((size_t)nnz + kThreads - 1) / kThreads), kThreads, 0, st>>>(m, ncols, nnz, ir, ic, flags);
    g_launches += 1;
    int h = 0;
    err = cudaMemcpyAsync(&h, flags, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (err == cudaSuccess) err = cudaStreamSynchronize(st);
    if (err != cudaSuccess) return (int)err;
    return h ? (int)cudaErrorInvalidValue : 0;
}

int bidmat_b200_sdoprow(int nrows, int ncols, int nnz, float *A, const int *Aic, const float *B, int len, int opn) {
    (void)nrows; (void)ncols;
    return sdop_common<float>(nnz, A, Aic, B, len, opn);
}

int bidmat_b200_sdopcol(int nrows, int ncols, int nnz, float *A, const int *Air, const float *B, int len, int opn) {
    (void)nrows; (void)ncols;
    return sdop_common<float>(nnz, A, Air, B, len, opn);
}

int bidmat_b200_sdoprow_f64(int nrows, int ncols, int nnz, double *A, const int *Aic, const double *B, int len, int opn) {
    (void)nrows; (void)ncols;
    return sdop_common<double>(nnz, A, Aic, B, len, opn);
}

int bidmat_b200_sdopcol_f64(int nrows, int ncols, int nnz, double *A, const int *Air, const double *B, int len, int opn) {
    (void)nrows; (void)ncols;
    return sdop_common<double>(nnz, A, Air, B, len, opn);
}

int bidmat_b200_spsum(int nrows, int ncols, int nnz, const int *Air, const int *Aic, const float *P, float *B, int n) {
    return spsum_impl<float>(nrows, ncols, nnz, Air, Aic, P, B, n);
}

int bidmat_b200_spsum_f64(int nrows, int ncols, int nnz, const int *Air, const int *Aic, const double *P, double *B,
                          int n) {
    return spsum_impl<double>(nrows, ncols, nnz, Air, Aic, P, B, n);
}

// C(nr x nc tile) += A(nr x kk tile) * S[broff:broff+kk, bcoff:bcoff+nc]       (transpose == 0)
// C(nr x nc tile) += A(nr x kk tile) * S[broff:broff+nc, bcoff:bcoff+kk]^T     (transpose != 0)
int bidmat_b200_dsmultTile(int nr, int nc, int kk, int nnz, const float *A, int lda, const float *Bdata,
                           const int *Bir, const int *Bic, int broff, int bcoff, float *C, int ldc, int transpose) {
    if (nr < 0 || nc < 0 || kk < 0 || nnz < 0 || lda < nr || ldc < nr) return (int)cudaErrorInvalidValue;
    if (nnz == 0 || nr == 0 || nc == 0 || kk == 0) return 0;
    if (!A || !Bdata || !Bir || !Bic || !C) return (int)cudaErrorInvalidValue;
    cudaStream_t st = cudaStreamPerThread;
    const size_t n_ = (size_t)nnz;
    const int ctiles = (int)((n_ + kCompactTile - 1) / kCompactTile);
    // rows and columns of S that the tile keeps
    const int nrt = transpose ? nc : kk, nct = transpose ? kk : nc;
    const bool aligned = is16(A) && is16(C) && (lda % 4 == 0) && (ldc % 4 == 0);
    const Shape s = pick_shape(nr, aligned);
    const int chunk_all = pick_chunk(nnz, s.lpv);
    const size_t part_floats = (size_t)max_chunks_for(nnz, s.lpv) * 2 * (size_t)nr;
    const int stiles = (int)((n_ + kSortTile - 1) / kSortTile);
    size_t need = 3 * pad256(n_ * 4) + pad256(((size_t)ctiles + 1) * 4) + pad256(part_floats * 4) + 4096;
    if (transpose) need += 6 * pad256(n_ * 4) + pad256((size_t)256 * stiles * 4) + pad256(256 * kSortScanSegs * 4);
    WorkspaceLease ws(need, st);
    if (ws.err != cudaSuccess) return (int)ws.err;
    int *trow = ws.take<int>(n_);
    int *tcol = ws.take<int>(n_);
    float *tval = ws.take<float>(n_);
    int *offs = ws.take<int>((size_t)ctiles + 1);
    float *part = ws.take<float>(part_floats);

    compact_count_kernel<<<ctiles, kCompactThreads, 0, st>>>(nnz, Bir, Bic, broff, nrt, bcoff, nct, offs);
    compact_scan_kernel<<<1, 1024, 0, st>>>(ctiles, offs);
    compact_scatter_kernel<float><<<ctiles, kCompactThreads, 0, st>>>(nnz, Bir, Bic, Bdata, broff, nrt, bcoff, nct, offs,
                                                                      trow, tcol, tval);
    g_launches += 3;
    int kept = 0;
    cudaError_t err = cudaMemcpyAsync(&kept, offs + ctiles, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (err == cudaSuccess) err = cudaStreamSynchronize(st);
    if (err != cudaSuccess) return (int)err;
    if (kept == 0) return (int)cudaGetLastError();
    const int chunk = pick_chunk(kept, s.lpv);
    if (!transpose) {
        // tile-relative columns are still non-decreasing: gather-accumulate directly
        err = launch_ga<float>(nr, kept, A, tval, trow, tcol, C, part, chunk, s, st, "tile_ga_chunk", -1, nullptr,
                               0xffffffffu, lda, ldc);
        return finish_sync(err, st);
    }
    // transposed tile: order the kept nonzeros by tile-relative row, then gather columns of A
    unsigned *keys[2] = {ws.take<unsigned>((size_t)kept), ws.take<unsigned>((size_t)kept)};
    int *cols[2] = {ws.take<int>((size_t)kept), ws.take<int>((size_t)kept)};
    float *vals[2] = {ws.take<float>((size_t)kept), ws.take<float>((size_t)kept)};
    int *counts = ws.take<int>((size_t)256 * stiles);
    int *totals = ws.take<int>(256 * kSortScanSegs);
    int rowbits = ceil_log2((unsigned long long)(nrt > 1 ? nrt : 2));
    const int cur = run_rowsort<float>(kept, (rowbits + 7) / 8, SortKeySpec{31, rowbits}, trow, tcol, tval, keys, cols,
                                       vals, nullptr, nullptr, nullptr, counts, totals, st);
    err = cudaGetLastError();
    if (err != cudaSuccess) return (int)err;
    err = launch_ga<float>(nr, kept, A, vals[cur], cols[cur], reinterpret_cast<const int *>(keys[cur]), C, part, chunk, s,
                           st, "tile_ga_chunk", -1, nullptr, 0xffffffffu, lda, ldc);
    return finish_sync(err, st);
}

long long bidmat_b200_workspace_bytes(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    std::lock_guard<std::mutex> g(g_pools[dev].mu);
    if (!g_pools[dev].pool) return 0;
    unsigned long long reserved = 0;
    if (cudaMemPoolGetAttribute(g_pools[dev].pool, cudaMemPoolAttrReservedMemCurrent, &reserved) != cudaSuccess) return 0;
    return (long long)reserved;
}

int bidmat_b200_release_workspace(void) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return (int)err;
    if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(g_pools[dev].mu);
    if (!g_pools[dev].pool) return 0;
    // blocks still leased by calls in flight stay; everything already returned goes back to the driver
    return (int)cudaMemPoolTrimTo(g_pools[dev].pool, 0);
}

int bidmat_b200_set_workspace_limit(long long bytes) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return (int)err;
    if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
    if (bytes < 0) return (int)cudaErrorInvalidValue;
    g_pools[dev].limit.store(bytes);
    return 0;
}

long long bidmat_b200_launch_count(void) { return g_launches.load(); }

int bidmat_b200_timing_enable(int on) {
    g_timing.store(on ? 1 : 0);
    return 0;
}

int bidmat_b200_timing_read(const char *label, double *total_ms, long long *count) {
    if (!label || !total_ms || !count) return (int)cudaErrorInvalidValue;
    std::lock_guard<std::mutex> g(g_span_mu);
    double tot = 0.0;
    long long c = 0;
    for (const TimedSpan &sp : g_spans) {
        if (strcmp(sp.label, label) != 0) continue;
        cudaError_t err = cudaEventSynchronize(sp.b);
        if (err != cudaSuccess) return (int)err;
        float ms = 0.f;
        err = cudaEventElapsedTime(&ms, sp.a, sp.b);
        if (err != cudaSuccess) return (int)err;
        tot += ms;
        c++;
    }
    *total_ms = tot;
    *count = c;
    return 0;
}

int bidmat_b200_timing_reset(void) {
    std::lock_guard<std::mutex> g(g_span_mu);
    for (const TimedSpan &sp : g_spans) {
        cudaEventDestroy(sp.a);
        cudaEventDestroy(sp.b);
    }
    g_spans.clear();
    return 0;
}

int bidmat_b200_version(void) { return 100; }

const char *bidmat_b200_error_string(int err) { return cudaGetErrorString((cudaError_t)err); }

}  // extern "C"
