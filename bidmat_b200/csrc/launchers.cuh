// Launch helpers shared by the translation units that drive the gather-accumulate
// and sampled-product kernels: kernel selection by the dense height, the fix-up
// launch and the row sort driver.
#pragma once
#include <type_traits>

#include "kernels.cuh"
#include "rowsort.cuh"
#include "host_common.cuh"
#include "workspace.cuh"

namespace bidmat {

// O[:, seg[j]] += val[j] * D[:, gidx[j]] with `part` holding 2*nchunks*k floats.
constexpr int kFastThreads = 128;

// k = vec*lpv*nt exactly with 16-byte vectors (4 floats / 2 doubles) and aligned operands:
// the predicate-free kernels apply.
inline bool fast_shape(int k, const Shape &s) { return s.vec > 1 && s.tiles == 1 && k == s.vec * s.lpv * s.nt; }

// `count` nonzeros are processed: the whole list (range == nullptr, count == nnz) or
// the slice [range[0], range[1]) read on the device.  The output column of a
// nonzero is seg & segmask.  S is float or double.
template <typename S>
cudaError_t launch_ga(int k, long long nnz, const S *D, const S *val, const int *gidx,
                      const int *seg, S *O, S *part, int chunk, const Shape &s,
                      cudaStream_t st, const char *label, long long count = -1,
                      const int *range = nullptr, unsigned segmask = 0xffffffffu, int ld_d = 0, int ld_o = 0) {
    constexpr int kWideVec = 16 / (int)sizeof(S);
    if (ld_d <= 0) ld_d = k;     // leading dimensions: k unless the operands are tiles of larger matrices
    if (ld_o <= 0) ld_o = k;
    if (count < 0) count = nnz;
    if (count == 0) return cudaSuccess;
    const long long nchunks = (count + chunk - 1) / chunk;
    dim3 grid(blocks_for(nchunks, s.lpv), s.tiles, 1);
    bool done = false;
    if (fast_shape(k, s) && ld_d == k && ld_o == k && !env_int("BIDMAT_B200_GENERIC", 0)) {
        const int wpb = kFastThreads / s.lpv;
        dim3 fgrid((unsigned)((nchunks + wpb - 1) / wpb), 1, 1);
        ScopedSpan sp(label, st);
#define CALL_FAST(LPV, NT, U, MINB)                                                                    \
    ga_chunk_fast_kernel<S, LPV, NT, U, kFastThreads, MINB><<<fgrid, kFastThreads, 0, st>>>(nnz, chunk, nchunks, D, val, \
                                                                                           gidx, seg, O, part, range, segmask)
        if (s.lpv == 8) { CALL_FAST(8, 1, 4, 0); }
        else if (s.lpv == 16) { CALL_FAST(16, 1, 4, 0); }
        else if (s.nt == 1) { CALL_FAST(32, 1, 4, 0); }
        else if (s.nt == 2) { CALL_FAST(32, 2, 2, 5); }
        else { CALL_FAST(32, 4, 1, 0); }
#undef CALL_FAST
        done = true;
    }
    if (!done) {
#define CALL_GA(VEC, LPV, NT)                                                                   \
    {                                                                                           \
        ScopedSpan sp(label, st);                                                               \
        ga_chunk_kernel<S, VEC, LPV, NT, 4><<<grid, kThreads, 0, st>>>(k, nnz, chunk, nchunks, D, val, \
                                                                       gidx, seg, O, part, range, \
                                                                       segmask, ld_d, ld_o, nullptr, 0u); \
    }
        DISPATCH_SHAPE(s, CALL_GA);
#undef CALL_GA
    }
    if (nchunks > 1) {
        ScopedSpan sp("ga_fixup", st);
#define CALL_FIX(VEC, LPV, NT) \
    ga_fixup_kernel<S, VEC, LPV, NT><<<grid, kThreads, 0, st>>>(k, nnz, chunk, nchunks, seg, O, part, range, segmask, ld_o);
        DISPATCH_SHAPE(s, CALL_FIX);
#undef CALL_FIX
    }
    g_launches += (nchunks > 1) ? 2 : 1;
    return cudaGetLastError();
}

template <typename S, bool ACCUM>
cudaError_t launch_dds(int k, long long nnz, const S *A, const S *B, const int *ir,
                       const int *ic, S *P, cudaStream_t st) {
    constexpr int kWideVec = 16 / (int)sizeof(S);
    const Shape s = pick_shape(k, is16(A) && is16(B), kWideVec);
    const int chunk = pick_chunk(nnz, s.lpv);
    const long long nchunks = (nnz + chunk - 1) / chunk;
    dim3 grid(blocks_for(nchunks, s.lpv), 1, 1);
    ScopedSpan sp("dds_chunk", st);
    bool done = false;
    // fp32: k = 128, 256; fp64: k = 64, 128, 256 (four vectors per lane, two nonzeros in flight)
    const int max_nt = std::is_same<S, float>::value ? 2 : 4;
    if (fast_shape(k, s) && s.lpv == 32 && s.nt <= max_nt && !env_int("BIDMAT_B200_GENERIC", 0)) {
        const int wpb = kFastThreads / 32;
        dim3 fgrid((unsigned)((nchunks + wpb - 1) / wpb), 1, 1);
        if (s.nt == 1)
            dds_chunk_fast_kernel<S, 1, 4, kFastThreads, ACCUM><<<fgrid, kFastThreads, 0, st>>>(nnz, chunk, nchunks, A, B, ir, ic, P);
        else if (s.nt == 2)
            dds_chunk_fast_kernel<S, 2, 4, kFastThreads, ACCUM><<<fgrid, kFastThreads, 0, st>>>(nnz, chunk, nchunks, A, B, ir, ic, P);
        else if constexpr (!std::is_same<S, float>::value)
            dds_chunk_fast_kernel<S, 4, 2, kFastThreads, ACCUM><<<fgrid, kFastThreads, 0, st>>>(nnz, chunk, nchunks, A, B, ir, ic, P);
        done = true;
    }
    if (!done) {
#define CALL_DDS(VEC, LPV, NT)                                                                  \
    dds_chunk_kernel<S, VEC, LPV, NT, 4, ACCUM><<<grid, kThreads, 0, st>>>(k, nnz, chunk, nchunks, A, B, \
                                                                           ir, ic, P);
        DISPATCH_SHAPE(s, CALL_DDS);
#undef CALL_DDS
    }
    g_launches += 1;
    return cudaGetLastError();
}

// A*S and DDS in one pass where the fused kernel applies (fp32, k = 128 / 256 / 512, aligned
// operands); returns false when it does not, and the caller runs the two operations separately.
inline bool launch_as_dds(int k, long long nnz, const float *A, const float *B, const float *val, const int *ir,
                          const int *ic, float *C, float *P, float *part, int chunk, cudaStream_t st, cudaError_t *err) {
    const Shape s = pick_shape(k, is16(A) && is16(B) && is16(C), 4);
    if (!fast_shape(k, s) || s.lpv != 32 || env_int("BIDMAT_B200_GENERIC", 0) || !env_int("BIDMAT_B200_FUSE_AS_DDS", 1))
        return false;
    const long long nchunks = (nnz + chunk - 1) / chunk;
    const int wpb = kFastThreads / 32;
    dim3 fgrid((unsigned)((nchunks + wpb - 1) / wpb), 1, 1);
    {
        ScopedSpan sp("dsmult_dds_chunk", st);
        if (s.nt == 1) as_dds_chunk_fast_kernel<1, 4, kFastThreads, 0><<<fgrid, kFastThreads, 0, st>>>(nnz, chunk, nchunks, A, B, val, ir, ic, C, part, P);
        else if (s.nt == 2) as_dds_chunk_fast_kernel<2, 2, kFastThreads, 5><<<fgrid, kFastThreads, 0, st>>>(nnz, chunk, nchunks, A, B, val, ir, ic, C, part, P);
        else as_dds_chunk_fast_kernel<4, 1, kFastThreads, 0><<<fgrid, kFastThreads, 0, st>>>(nnz, chunk, nchunks, A, B, val, ir, ic, C, part, P);
    }
    if (nchunks > 1) {
        ScopedSpan sp("ga_fixup", st);
        dim3 grid(blocks_for(nchunks, 32), 1, 1);
        if (s.nt == 1) ga_fixup_kernel<float, 4, 32, 1><<<grid, kThreads, 0, st>>>(k, nnz, chunk, nchunks, ic, C, part, nullptr, 0xffffffffu, k);
        else if (s.nt == 2) ga_fixup_kernel<float, 4, 32, 2><<<grid, kThreads, 0, st>>>(k, nnz, chunk, nchunks, ic, C, part, nullptr, 0xffffffffu, k);
        else ga_fixup_kernel<float, 4, 32, 4><<<grid, kThreads, 0, st>>>(k, nnz, chunk, nchunks, ic, C, part, nullptr, 0xffffffffu, k);
    }
    g_launches += (nchunks > 1) ? 2 : 1;
    *err = cudaGetLastError();
    return true;
}

// Sorts the nonzero list (ir, ic, v) by key (see rowsort.cuh) in `passes` 8-bit
// passes.  Intermediate results ping-pong between the two scratch buffer sets;
// when out_* are given the last pass writes there.  Returns the index of the
// scratch set holding the result, or -1 when it went to out_*.
template <typename S>
int run_rowsort(int nnz, int passes, SortKeySpec ks, const int *ir, const int *ic, const S *v,
                unsigned *const keys[2], int *const cols[2], S *const vals[2], unsigned *out_keys,
                int *out_cols, S *out_vals, int *counts, int *totals, cudaStream_t st) {
    static std::once_flag smem_once[kMaxDevices];
    {
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= kMaxDevices) dev = 0;
        std::call_once(smem_once[dev], [] {
            cudaFuncSetAttribute(sort_scatter_kernel<true, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SortSmem<S>));
            cudaFuncSetAttribute(sort_scatter_kernel<false, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SortSmem<S>));
        });
    }
    const int ntiles = (int)(((size_t)nnz + kSortTile - 1) / kSortTile);
    const int tps = (ntiles + kSortScanSegs - 1) / kSortScanSegs;   // tiles per scan segment
    int cur = 0;   // scratch set holding the output of the last pass
    ScopedSpan sp("dsmultT_rowsort", st);
    for (int p = 0; p < passes; p++) {
        const int shift = 8 * p;
        const bool to_user = (p == passes - 1) && out_keys != nullptr;
        const int out = (p == 0) ? 0 : 1 - cur;
        unsigned *ko = to_user ? out_keys : keys[out];
        int *co = to_user ? out_cols : cols[out];
        S *vo = to_user ? out_vals : vals[out];
        {
            ScopedSpan sp1("sort_hist", st);
            if (p == 0) {
                sort_hist_kernel<true><<<ntiles, kSortThreads, 0, st>>>(nnz, ntiles, shift, ks, nullptr, ir, ic, counts);
            } else {
                sort_hist_kernel<false><<<ntiles, kSortThreads, 0, st>>>(nnz, ntiles, shift, ks, keys[cur], nullptr, nullptr, counts);
            }
        }
        {
            ScopedSpan sp2("sort_scan", st);
            sort_scan_kernel<<<dim3(kSortScanSegs, 256), kSortThreads, 0, st>>>(ntiles, tps, counts, totals);
            sort_digit_base_kernel<<<1, 256, 0, st>>>(totals);
        }
        {
            ScopedSpan sp3("sort_scatter", st);
            if (p == 0) {
                sort_scatter_kernel<true, S><<<ntiles, kSortThreads, sizeof(SortSmem<S>), st>>>(
                    nnz, ntiles, shift, ks, nullptr, ir, ic, v, counts, totals, tps, ko, co, vo);
            } else {
                sort_scatter_kernel<false, S><<<ntiles, kSortThreads, sizeof(SortSmem<S>), st>>>(
                    nnz, ntiles, shift, ks, keys[cur], nullptr, cols[cur], vals[cur], counts, totals, tps, ko, co, vo);
            }
        }
        g_launches += 4;
        cur = to_user ? -1 : out;
    }
    return cur;
}

// How B*^S cuts the columns of the dense operand into L2-sized blocks and how many
// 8-bit sort passes the key (column block, row) then needs.
struct BlockLayout {
    int colshift;     // column block of a nonzero = column >> colshift (31: one block)
    int nblocks;
    int rowbits;      // low key bits holding the row
    int passes;       // radix passes over the key
    unsigned rowmask;
};

// When the dense operand (ncols columns of k elements of `elem` bytes) is much
// larger than L2, the nonzeros are ordered by (column block, row) so that the
// gathers of one block stay L2-resident; the blocks are then processed one after
// the other.  `rows` is the height of the sparse matrix when known (0: 2^rowbits is
// assumed by the cost model); `max_keybits` bounds row bits + block bits.  Returns
// false when the row index does not fit the key.
inline bool choose_block_layout(int k, int ncols, long long nnz, size_t elem, int rowbits, double rows,
                                int max_keybits, BlockLayout *out) {
    if (rowbits < 1) rowbits = 1;
    if (rowbits > 31 || rowbits > max_keybits) return false;
    const size_t dense_bytes = (size_t)ncols * (size_t)k * elem;
    size_t l2_bytes = 96u << 20;
    {
        int dev = 0, l2 = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev) == cudaSuccess && l2 > 0)
            l2_bytes = (size_t)l2;
    }
    // block = half of L2 unless BIDMAT_B200_COLBLOCK_MB says otherwise (0 disables);
    // an operand up to 1.5 x L2 is left in one piece (measured: splitting a 128 MB
    // operand in two costs more in extra output passes than it gains in hits).
    const int block_mb = env_int("BIDMAT_B200_COLBLOCK_MB", -1);
    const size_t block_bytes = block_mb >= 0 ? ((size_t)block_mb << 20) : l2_bytes / 2;
    int colshift = 31;
    const int forced_cols = env_int("BIDMAT_B200_COLBLOCK_COLS", 0);   // tests force tiny blocks
    if (forced_cols > 0) {
        colshift = 0;
        while ((2 << colshift) <= forced_cols) colshift++;
    } else if (block_bytes > 0 && dense_bytes > l2_bytes + l2_bytes / 2) {
        // columns per block: the power of two nearest to block_bytes / column bytes
        size_t cols_per_block = block_bytes / ((size_t)k * elem);
        colshift = 0;
        while ((2ull << colshift) <= cols_per_block) colshift++;
        if (cols_per_block * 1000 >= (1ull << colshift) * 1414) colshift++;
    }
    int nblocks = (colshift >= 31) ? 1 : (((ncols - 1) >> colshift) + 1);
    while (nblocks > 1 && (rowbits + ceil_log2((unsigned long long)nblocks) > max_keybits || nblocks > 1023)) {
        colshift++;
        nblocks = ((ncols - 1) >> colshift) + 1;
    }
    // Is splitting worth it?  Unsplit, about every gather misses L2: nnz*k*elem bytes of
    // DRAM reads.  Split, the operand is read once but every block re-reads and re-writes
    // the output rows it touches (at most all of them) and the sort may need one more
    // pass over the nonzero list.  Split only for a clear win; tests that force a block
    // size skip the model.
    if (nblocks > 1 && forced_cols <= 0) {
        const double colbytes = (double)elem * k;
        if (rows <= 0.0) rows = (double)(1ull << rowbits);
        const double unsplit = (double)nnz * colbytes;
        const int extra_pass = ((rowbits + ceil_log2((unsigned long long)nblocks) + 7) / 8) - ((rowbits + 7) / 8);
        const double split = (double)dense_bytes + (double)nblocks * rows * 2.0 * colbytes +
                             2.0 * (8.0 + elem) * nnz * extra_pass;
        if (split > 0.6 * unsplit) nblocks = 1;
    }
    if (nblocks <= 1) { colshift = 31; nblocks = 1; }
    const int keybits = rowbits + (nblocks > 1 ? ceil_log2((unsigned long long)nblocks) : 0);
    out->colshift = colshift;
    out->nblocks = nblocks;
    out->rowbits = rowbits;
    out->passes = (keybits + 7) / 8;
    out->rowmask = (rowbits >= 32) ? 0xffffffffu : ((1u << rowbits) - 1u);
    return true;
}

}  // namespace bidmat
