// Prepared transposed product: bidmat_b200_dsmultT_plan_create sorts the
// structure of a sparse matrix once (what bidmat_b200_dsmultT does on every
// call) and keeps the result behind an explicit handle; bidmat_b200_dsmultT_planned
// then runs B*^S for any values on that structure without sorting and without a
// host round trip.  BIDMat keeps derived structure on the matrix object in the same
// way: GSMat.fromSMat computes the per-nonzero columns once
// (src/main/scala/BIDMat/GSMat.scala:620-647), and DDS copies the pattern of its
// sparse argument into its result (GSMat.scala:656-661), so the plan of S serves
// every G = B *^ DDS(A,B,S) of a factorisation loop.
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>
#include <cstdint>
#include <vector>

#include "../../include/bidmat_b200.h"
#include "launchers.cuh"
#include "plan_kernels.cuh"

using namespace bidmat;

struct bidmat_b200_plan {
    unsigned magic = 0;
    int dev = 0;
    int k = 0, ncols = 0, nnz = 0, m = 0, elem = 4;
    BlockLayout lay{};
    // device arrays owned by the plan
    unsigned *keys = nullptr;      // sorted (column block << rowbits) | row, bit 31 = first block of the row
    int *cols = nullptr;           // source column per sorted nonzero
    int *perm = nullptr;           // original position per sorted nonzero
    int *inv = nullptr;            // sorted position per original nonzero (BIDMAT_B200_PLAN_SCATTER=1 only)
    int4 *desc = nullptr;          // chunk descriptors, all blocks
    int4 *runs = nullptr;          // split runs {key, first slot, pieces, 0}, ordered by (row, block)
    int4 *groups = nullptr;        // rows with split runs {row, first run, number of runs, 0}
    int *clear_rows = nullptr;     // rows cleared by an overwriting call (first run is split)
    unsigned *touched = nullptr;   // bitmap of the rows named by at least one nonzero
    void *part = nullptr;          // slots of the split runs, nslots * k elements
    int *mismatch = nullptr;       // result of plan_verify
    std::vector<int> block_c0, block_nch;
    // host copies for running a single-block plan in row ranges (bidmat_b200_plan_row_parts)
    std::vector<int> h_chunk_row;      // row of the first nonzero of a chunk, -1 when the chunk starts inside a row
    std::vector<int> h_group_row, h_group_run0;
    std::vector<int> part_chunk, part_run, part_group, part_row, part_clear;   // bounds per part, nparts + 1 entries each
    std::vector<int> h_clear_rows;  // host copy of clear_rows (ascending in a single-block plan)
    int nchunks = 0, nruns = 0, ngroups = 0, nslots = 0, nclear = 0;
    long long touched_rows = 0;
    long long row_runs = 0;        // runs of equal (column block, row): each one updates its output column once
    size_t bytes = 0;
};

namespace {

constexpr unsigned kPlanMagic = 0xB1D0A7u;
constexpr unsigned kStoreBit = 0x80000000u;

template <typename T> cudaError_t plan_alloc(bidmat_b200_plan *p, T **out, size_t count) {
    *out = nullptr;
    if (count == 0) count = 1;
    cudaError_t err = cudaMalloc(reinterpret_cast<void **>(out), count * sizeof(T));
    if (err == cudaSuccess) p->bytes += count * sizeof(T);
    else { *out = nullptr; (void)cudaGetLastError(); }
    return err;
}

void plan_free(bidmat_b200_plan *p) {
    cudaFree(p->keys); cudaFree(p->cols); cudaFree(p->perm); cudaFree(p->inv); cudaFree(p->desc); cudaFree(p->runs); cudaFree(p->groups);
    cudaFree(p->clear_rows); cudaFree(p->touched); cudaFree(p->part); cudaFree(p->mismatch);
    p->magic = 0;
    delete p;
}

bool plan_ok(const bidmat_b200_plan *p) {
    if (!p || p->magic != kPlanMagic) return false;
    int dev = -1;
    return cudaGetDevice(&dev) == cudaSuccess && dev == p->dev;
}

#define PLAN_CK(expr)                                   \
    do {                                                \
        cudaError_t e_ = (expr);                        \
        if (e_ != cudaSuccess) { plan_free(p); return (int)e_; } \
    } while (0)

int plan_create(int k, int ncols, int nnz, int m, const int *Bir, const int *Bic, int elem, cudaStream_t st,
                bidmat_b200_plan **out) {
    if (!out) return (int)cudaErrorInvalidValue;
    *out = nullptr;
    if (k <= 0 || ncols <= 0 || nnz <= 0 || m <= 0 || !Bir || !Bic || (elem != 4 && elem != 8))
        return (int)cudaErrorInvalidValue;
    bidmat_b200_plan *p = new bidmat_b200_plan;
    p->k = k; p->ncols = ncols; p->nnz = nnz; p->m = m; p->elem = elem;
    PLAN_CK(cudaGetDevice(&p->dev));
    // bit 31 of the key is the first-block mark, so row bits + block bits <= 31
    if (!choose_block_layout(k, ncols, nnz, (size_t)elem, ceil_log2((unsigned long long)m), (double)m, 31, &p->lay)) {
        plan_free(p);
        return (int)cudaErrorInvalidValue;
    }
    const BlockLayout lay = p->lay;
    const size_t n = (size_t)nnz;
    PLAN_CK(plan_alloc(p, &p->keys, n));
    PLAN_CK(plan_alloc(p, &p->cols, n));
    PLAN_CK(plan_alloc(p, &p->perm, n));
    PLAN_CK(plan_alloc(p, &p->mismatch, 1));

    // ---- sort (key, column, position); the scratch goes back to the pool before returning
    std::vector<int> h_off((size_t)lay.nblocks + 1);
    std::vector<int> h_first;
    {
        const int ntiles = (int)((n + kSortTile - 1) / kSortTile);
        const size_t need = 6 * pad256(n * 4) + pad256((size_t)256 * ntiles * 4) + pad256(256 * kSortScanSegs * 4) +
                            pad256(4096) + pad256((size_t)m * 4) + 8192;
        WorkspaceLease ws(need, st);
        PLAN_CK(ws.err);
        unsigned *keys[2] = {ws.take<unsigned>(n), ws.take<unsigned>(n)};
        int *cols[2] = {ws.take<int>(n), ws.take<int>(n)};
        int *vals[2] = {ws.take<int>(n), ws.take<int>(n)};
        int *counts = ws.take<int>((size_t)256 * ntiles);
        int *totals = ws.take<int>(256 * kSortScanSegs);
        int *offsets = ws.take<int>(1024);
        int *first_block = ws.take<int>((size_t)m);
        unsigned long long *d_nruns = ws.take<unsigned long long>(1);
        run_rowsort<int>(nnz, lay.passes, SortKeySpec{lay.colshift, lay.rowbits}, Bir, Bic, nullptr, keys, cols, vals,
                         p->keys, p->cols, p->perm, counts, totals, st);
        PLAN_CK(cudaGetLastError());
        block_offsets_kernel<<<(lay.nblocks + 256) / 256, 256, 0, st>>>(nnz, lay.nblocks, lay.rowbits, p->keys, offsets);
        PLAN_CK(cudaMemsetAsync(first_block, 0x7f, (size_t)m * 4, st));      // kNoBlock in every entry
        PLAN_CK(cudaMemsetAsync(d_nruns, 0, sizeof(unsigned long long), st));
        plan_first_block_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(nnz, p->keys, lay.rowbits, lay.rowmask,
                                                                           first_block, d_nruns);
        g_launches += 2;
        h_first.resize((size_t)m);
        PLAN_CK(cudaMemcpyAsync(h_off.data(), offsets, sizeof(int) * (lay.nblocks + 1), cudaMemcpyDeviceToHost, st));
        PLAN_CK(cudaMemcpyAsync(h_first.data(), first_block, sizeof(int) * (size_t)m, cudaMemcpyDeviceToHost, st));
        unsigned long long h_nruns = 0;
        PLAN_CK(cudaMemcpyAsync(&h_nruns, d_nruns, sizeof(h_nruns), cudaMemcpyDeviceToHost, st));
        PLAN_CK(cudaStreamSynchronize(st));
        p->row_runs = (long long)h_nruns;
    }

    if (env_int("BIDMAT_B200_PLAN_SCATTER", 0)) {
        PLAN_CK(plan_alloc(p, &p->inv, n));
        plan_invert_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(nnz, p->perm, p->inv);
        g_launches += 1;
        PLAN_CK(cudaGetLastError());
    }

    // ---- chunk grid of every block
    std::vector<int> T((size_t)lay.nblocks, 0);
    p->block_c0.assign((size_t)lay.nblocks, 0);
    p->block_nch.assign((size_t)lay.nblocks, 0);
    int total = 0;
    for (int b = 0; b < lay.nblocks; b++) {
        const long long count = (long long)h_off[b + 1] - h_off[b];
        p->block_c0[b] = total;
        if (count <= 0) continue;
        // half the chunk length of the unprepared path (twice the chunks per launch): measured 0.3 ms
        // less over the 16 launches of the LDA configuration; boundaries move to row boundaries anyway,
        // so no rounding to the worker width
        T[b] = pick_chunk((count + 1) / 2, 1);
        p->block_nch[b] = (int)((count + T[b] - 1) / T[b]);
        total += p->block_nch[b];
    }
    p->nchunks = total;
    const size_t nb_entries = (size_t)total + (size_t)lay.nblocks;      // nch + 1 boundaries per block
    std::vector<int> h_start(nb_entries);
    std::vector<unsigned> h_kfirst(nb_entries), h_kprev(nb_entries);
    {
        WorkspaceLease ws(3 * pad256(nb_entries * 4) + 1024, st);
        PLAN_CK(ws.err);
        int *d_start = ws.take<int>(nb_entries);
        unsigned *d_first = ws.take<unsigned>(nb_entries);
        unsigned *d_prev = ws.take<unsigned>(nb_entries);
        for (int b = 0; b < lay.nblocks; b++) {
            const int nch = p->block_nch[b];
            if (nch == 0) continue;
            const size_t e0 = (size_t)p->block_c0[b] + b;
            plan_bounds_kernel<<<(nch + 256) / 256, 256, 0, st>>>(h_off[b], h_off[b + 1], T[b], nch, p->keys,
                                                                  d_start + e0, d_first + e0, d_prev + e0);
            g_launches += 1;
        }
        PLAN_CK(cudaGetLastError());
        PLAN_CK(cudaMemcpyAsync(h_start.data(), d_start, nb_entries * 4, cudaMemcpyDeviceToHost, st));
        PLAN_CK(cudaMemcpyAsync(h_kfirst.data(), d_first, nb_entries * 4, cudaMemcpyDeviceToHost, st));
        PLAN_CK(cudaMemcpyAsync(h_kprev.data(), d_prev, nb_entries * 4, cudaMemcpyDeviceToHost, st));
        PLAN_CK(cudaStreamSynchronize(st));
    }

    // ---- descriptors, slots of the split runs, rows an overwriting call has to clear
    std::vector<int4> h_desc((size_t)total);
    std::vector<int4> h_runs;
    std::vector<unsigned char> h_nostore((size_t)m, 0);
    std::vector<int> h_clear;
    int slot = 0;
    for (int b = 0; b < lay.nblocks; b++) {
        const int nch = p->block_nch[b];
        const size_t e0 = (size_t)p->block_c0[b] + b;
        for (int c = 0; c < nch; c++) {
            const size_t e = e0 + c;
            const bool head = c > 0 && h_kprev[e] == h_kfirst[e];
            const bool tail = c + 1 < nch && h_kprev[e + 1] == h_kfirst[e + 1];
            const bool whole = head && tail && h_kfirst[e] == h_kprev[e + 1];
            int4 d;
            d.x = h_start[e];
            d.y = h_start[e + 1];
            d.z = head ? slot++ : -1;
            if (head) h_runs.back().z++;
            if (tail && !whole) {
                d.w = slot++;
                h_runs.push_back(make_int4((int)h_kprev[e + 1], d.w, 1, 0));
                const unsigned key = h_kprev[e + 1];
                const unsigned row = key & lay.rowmask;
                if ((int)(key >> lay.rowbits) == h_first[row] && !h_nostore[row]) {
                    h_nostore[row] = 1;
                    h_clear.push_back((int)row);
                }
            } else {
                d.w = tail ? -2 : -1;
            }
            h_desc[(size_t)p->block_c0[b] + c] = d;
            p->h_chunk_row.push_back(head ? -1 : (int)(h_kfirst[e] & lay.rowmask));
        }
    }
    p->nslots = slot;
    p->nruns = (int)h_runs.size();
    // Runs were listed block after block; a row split in several blocks has several.  Bring the
    // runs of one row together, blocks ascending (stable sort by row), and list the rows.
    std::stable_sort(h_runs.begin(), h_runs.end(), [&](const int4 &a, const int4 &b) {
        return ((unsigned)a.x & lay.rowmask) < ((unsigned)b.x & lay.rowmask);
    });
    std::vector<int4> h_groups;
    for (size_t r = 0; r < h_runs.size(); r++) {
        const int row = (int)((unsigned)h_runs[r].x & lay.rowmask);
        if (h_groups.empty() || h_groups.back().x != row) h_groups.push_back(make_int4(row, (int)r, 0, 0));
        h_groups.back().z++;
    }
    p->ngroups = (int)h_groups.size();
    p->h_group_row.resize(h_groups.size());
    p->h_group_run0.resize(h_groups.size());
    for (size_t g = 0; g < h_groups.size(); g++) { p->h_group_row[g] = h_groups[g].x; p->h_group_run0[g] = h_groups[g].y; }
    p->nclear = (int)h_clear.size();
    p->h_clear_rows = h_clear;
    for (int r = 0; r < m; r++) p->touched_rows += (h_first[r] != kNoBlock);

    PLAN_CK(plan_alloc(p, &p->desc, (size_t)total));
    PLAN_CK(plan_alloc(p, &p->runs, h_runs.size()));
    PLAN_CK(plan_alloc(p, &p->groups, h_groups.size()));
    PLAN_CK(plan_alloc(p, &p->clear_rows, h_clear.size()));
    PLAN_CK(plan_alloc(p, &p->touched, ((size_t)m + 31) / 32));
    {
        char *part = nullptr;
        PLAN_CK(plan_alloc(p, &part, (size_t)slot * (size_t)k * (size_t)elem));
        p->part = part;
    }
    PLAN_CK(cudaMemcpyAsync(p->desc, h_desc.data(), (size_t)total * sizeof(int4), cudaMemcpyHostToDevice, st));
    if (!h_runs.empty())
        PLAN_CK(cudaMemcpyAsync(p->runs, h_runs.data(), h_runs.size() * sizeof(int4), cudaMemcpyHostToDevice, st));
    if (!h_groups.empty())
        PLAN_CK(cudaMemcpyAsync(p->groups, h_groups.data(), h_groups.size() * sizeof(int4), cudaMemcpyHostToDevice, st));
    if (!h_clear.empty())
        PLAN_CK(cudaMemcpyAsync(p->clear_rows, h_clear.data(), h_clear.size() * sizeof(int), cudaMemcpyHostToDevice, st));
    {
        // first-block marks and the touched-row bitmap need first_block and no_store on the device once more
        WorkspaceLease ws(pad256((size_t)m * 4) + pad256((size_t)m) + 1024, st);
        PLAN_CK(ws.err);
        int *first_block = ws.take<int>((size_t)m);
        unsigned char *no_store = ws.take<unsigned char>((size_t)m);
        PLAN_CK(cudaMemcpyAsync(first_block, h_first.data(), (size_t)m * 4, cudaMemcpyHostToDevice, st));
        PLAN_CK(cudaMemcpyAsync(no_store, h_nostore.data(), (size_t)m, cudaMemcpyHostToDevice, st));
        plan_mark_first_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(nnz, p->keys, lay.rowbits, lay.rowmask,
                                                                          first_block, no_store);
        plan_touched_kernel<<<(unsigned)(((size_t)m + 255) / 256), 256, 0, st>>>(m, first_block, p->touched);
        g_launches += 2;
        PLAN_CK(cudaGetLastError());
        PLAN_CK(cudaStreamSynchronize(st));     // the host vectors above must outlive the copies
    }
    p->magic = kPlanMagic;
    *out = p;
    return 0;
}

// part < 0: the whole product.  part >= 0: only the row range `part` of a single-block plan
// (bidmat_b200_plan_row_parts): its chunks, then the fix-up of the split rows inside it.
template <typename S>
int plan_run(bidmat_b200_plan *p, int k, int ncols, int nnz, const S *A, const S *Bdata, S *C, int flags,
             cudaStream_t st, int part_index = -1) {
    if (!plan_ok(p)) return (int)cudaErrorInvalidValue;
    if (part_index >= 0 && (p->part_chunk.empty() || part_index + 1 >= (int)p->part_chunk.size()))
        return (int)cudaErrorInvalidValue;
    if (p->elem != (int)sizeof(S) || k != p->k || ncols != p->ncols || nnz != p->nnz) return (int)cudaErrorInvalidValue;
    if (!A || !Bdata || !C) return (int)cudaErrorInvalidValue;
    if (flags & ~BIDMAT_B200_PLAN_OVERWRITE) return (int)cudaErrorInvalidValue;
    constexpr int kWideVec = 16 / (int)sizeof(S);
    const Shape s = pick_shape(k, is16(A) && is16(C), kWideVec);
    const size_t n = (size_t)nnz;
    const unsigned storebit = (flags & BIDMAT_B200_PLAN_OVERWRITE) ? kStoreBit : 0u;
    const unsigned segmask = p->lay.rowmask;
    S *part = static_cast<S *>(p->part);
    const int *seg = reinterpret_cast<const int *>(p->keys);

    // The predicate-free float kernel reads the values through the stored positions itself
    // (BIDMAT_B200_PLAN_FUSED=0 switches that off); the double one and every other shape first
    // bring them into the plan's order with one gather pass into scratch.
    const bool fast = fast_shape(k, s) && !env_int("BIDMAT_B200_GENERIC", 0);
    const bool fused = fast && std::is_same<S, float>::value && env_int("BIDMAT_B200_PLAN_FUSED", 1) != 0;
    if (part_index >= 0 && !fused) return (int)cudaErrorNotSupported;   // parts need the kernel that reads the values in place
    WorkspaceLease ws(fused ? 256 : pad256(n * sizeof(S)) + 256, st);
    if (ws.err != cudaSuccess) return (int)ws.err;
    S *vals = fused ? nullptr : ws.take<S>(n);
    if (!fused) {
        ScopedSpan sp("dsmultT_permute", st);
        if (p->inv) plan_scatter_kernel<S><<<148 * 16, 256, 0, st>>>((long long)nnz, p->inv, Bdata, vals);
        else plan_permute_kernel<S><<<148 * 16, 256, 0, st>>>((long long)nnz, p->perm, Bdata, vals);
        g_launches += 1;
    }
    {
        // rows whose first run is split accumulate through the fix-up: an overwriting call clears them
        // first (a row range clears its own, so the ranges may run in any order)
        int clear0 = 0, nclear = p->nclear;
        if (part_index >= 0) {
            clear0 = p->part_clear[part_index];
            nclear = p->part_clear[part_index + 1] - clear0;
        }
        if (storebit && nclear > 0) {
            plan_clear_rows_kernel<S><<<(unsigned)(((size_t)nclear * 32 + 255) / 256), 256, 0, st>>>(k, nclear,
                                                                                                     p->clear_rows + clear0, C);
            g_launches += 1;
        }
    }
    const bool prefetch = env_int("BIDMAT_B200_PLAN_PREFETCH", 1) != 0;
    for (int b = 0; b < p->lay.nblocks; b++) {
        int nch = p->block_nch[b];
        const int4 *desc = p->desc + p->block_c0[b];
        if (part_index >= 0) {           // single block: the chunks of this row range
            desc += p->part_chunk[part_index];
            nch = p->part_chunk[part_index + 1] - p->part_chunk[part_index];
        }
        if (nch == 0) continue;
        ScopedSpan sp("dsmultT_ga_chunk", st);
        bool done = false;
        if (fast) {
            const int wpb = kFastThreads / s.lpv;
            const unsigned fgrid = (unsigned)((nch + wpb - 1) / wpb);
#define CALL_PLAN(LPV, NT, U, MINB)                                                                                \
    do {                                                                                                           \
        if constexpr (std::is_same<S, float>::value) {                                                             \
            if (fused) {                                                                                           \
                ga_plan_fast_kernel<S, LPV, NT, U, kFastThreads, MINB, true, true><<<fgrid, kFastThreads, 0, st>>>( \
                    nch, desc, A, Bdata, p->perm, p->cols, seg, C, part, segmask, storebit);                       \
                break;                                                                                             \
            }                                                                                                      \
        }                                                                                                          \
        if (prefetch)                                                                                              \
            ga_plan_fast_kernel<S, LPV, NT, U, kFastThreads, MINB, true, false><<<fgrid, kFastThreads, 0, st>>>(   \
                nch, desc, A, vals, nullptr, p->cols, seg, C, part, segmask, storebit);                            \
        else                                                                                                       \
            ga_plan_fast_kernel<S, LPV, NT, U, kFastThreads, MINB, false, false><<<fgrid, kFastThreads, 0, st>>>(  \
                nch, desc, A, vals, nullptr, p->cols, seg, C, part, segmask, storebit);                            \
    } while (0)
            if (s.lpv == 8) CALL_PLAN(8, 1, 4, 0);
            else if (s.lpv == 16) CALL_PLAN(16, 1, 4, 0);
            else if (s.nt == 1) CALL_PLAN(32, 1, 4, 0);
            else if (s.nt == 2) {
                // five CTAs of 128 threads per SM (<= 96 registers, a few spilled words) against
                // four without spills: BIDMAT_B200_PLAN_MINB picks, default 5 as for A*S
                if (env_int("BIDMAT_B200_PLAN_MINB", 5) == 4) CALL_PLAN(32, 2, 2, 4);
                else CALL_PLAN(32, 2, 2, 5);
            }
            else CALL_PLAN(32, 4, 1, 0);
#undef CALL_PLAN
            done = true;
        }
        if (!done) {
            dim3 grid(blocks_for(nch, s.lpv), s.tiles, 1);
#define CALL_GA(VEC, LPV, NT)                                                                                  \
    ga_chunk_kernel<S, VEC, LPV, NT, 4><<<grid, kThreads, 0, st>>>(k, (long long)nnz, 0, (long long)nch, A, vals, \
                                                                   p->cols, seg, C, part, nullptr, segmask, k, k, \
                                                                   desc, storebit)
            DISPATCH_SHAPE(s, CALL_GA);
#undef CALL_GA
        }
        g_launches += 1;
    }
    int run0 = 0, nruns = p->nruns, group0 = 0, ngroups = p->ngroups;
    if (part_index >= 0) {
        run0 = p->part_run[part_index]; nruns = p->part_run[part_index + 1] - run0;
        group0 = p->part_group[part_index]; ngroups = p->part_group[part_index + 1] - group0;
    }
    if (nruns > 0) {
        ScopedSpan sp("ga_fixup", st);
        dim3 grid(blocks_for(nruns, s.lpv), s.tiles, 1);
        dim3 ggrid(blocks_for(ngroups, s.lpv), s.tiles, 1);
#define CALL_FIX(VEC, LPV, NT)                                                                              \
    do {                                                                                                    \
        plan_fixup_runs_kernel<S, VEC, LPV, NT><<<grid, kThreads, 0, st>>>(k, nruns, p->runs + run0, part); \
        plan_fixup_rows_kernel<S, VEC, LPV, NT><<<ggrid, kThreads, 0, st>>>(k, ngroups, p->groups + group0, p->runs, C, \
                                                                            part, segmask);                 \
    } while (0)
        DISPATCH_SHAPE(s, CALL_FIX);
#undef CALL_FIX
        g_launches += 2;
    }
    return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

int bidmat_b200_dsmultT_plan_create(int nrows, int ncols, int nnz, int m, const int *Bir, const int *Bic,
                                    int elem_bytes, bidmat_stream_t stream, bidmat_b200_plan_t *plan) {
    return plan_create(nrows, ncols, nnz, m, Bir, Bic, elem_bytes, as_stream(stream), plan);
}

int bidmat_b200_dsmultT_planned(bidmat_b200_plan_t plan, int nrows, int ncols, int nnz, const float *A,
                                const float *Bdata, float *C, int flags, bidmat_stream_t stream) {
    return plan_run<float>(plan, nrows, ncols, nnz, A, Bdata, C, flags, as_stream(stream));
}

int bidmat_b200_dsmultT_planned_f64(bidmat_b200_plan_t plan, int nrows, int ncols, int nnz, const double *A,
                                    const double *Bdata, double *C, int flags, bidmat_stream_t stream) {
    return plan_run<double>(plan, nrows, ncols, nnz, A, Bdata, C, flags, as_stream(stream));
}

int bidmat_b200_plan_row_parts(bidmat_b200_plan_t p, int nparts, int *row_bounds) {
    if (!p || p->magic != kPlanMagic || nparts < 1 || !row_bounds) return (int)cudaErrorInvalidValue;
    if (p->lay.nblocks != 1 || p->nchunks < nparts) return (int)cudaErrorNotSupported;
    // Part boundaries at chunks that start a new row (rows ascend through the single block), near
    // equal chunk counts; the runs and groups of a part are those of its rows (both lists ascend by row).
    std::vector<int> chunk(1, 0), row(1, 0);
    for (int i = 1; i < nparts; i++) {
        int c = (int)((long long)p->nchunks * i / nparts);
        if (c <= chunk.back()) c = chunk.back() + 1;
        while (c < p->nchunks && p->h_chunk_row[(size_t)c] < 0) c++;
        if (c >= p->nchunks) break;
        chunk.push_back(c);
        row.push_back(p->h_chunk_row[(size_t)c]);
    }
    const int actual = (int)chunk.size();
    chunk.push_back(p->nchunks);
    row.push_back(p->m);
    std::vector<int> grp(1, 0), run(1, 0), clr(1, 0);
    for (int i = 1; i <= actual; i++) {
        clr.push_back((int)(std::lower_bound(p->h_clear_rows.begin(), p->h_clear_rows.end(), row[(size_t)i]) -
                            p->h_clear_rows.begin()));
        const int g = (int)(std::lower_bound(p->h_group_row.begin(), p->h_group_row.end(), row[(size_t)i]) -
                            p->h_group_row.begin());
        grp.push_back(g);
        run.push_back(g < p->ngroups ? p->h_group_run0[(size_t)g] : p->nruns);
    }
    p->part_chunk = chunk; p->part_row = row; p->part_group = grp; p->part_run = run; p->part_clear = clr;
    for (int i = 0; i <= actual; i++) row_bounds[i] = row[(size_t)i];
    for (int i = actual + 1; i <= nparts; i++) row_bounds[i] = p->m;
    return actual == nparts ? 0 : (int)cudaErrorNotSupported;
}

int bidmat_b200_dsmultT_planned_part(bidmat_b200_plan_t plan, int nrows, int ncols, int nnz, const float *A,
                                     const float *Bdata, float *C, int flags, int part, bidmat_stream_t stream) {
    if (part < 0) return (int)cudaErrorInvalidValue;
    return plan_run<float>(plan, nrows, ncols, nnz, A, Bdata, C, flags, as_stream(stream), part);
}

int bidmat_b200_plan_verify(bidmat_b200_plan_t p, int ncols, int nnz, const int *Bir, const int *Bic,
                            bidmat_stream_t stream) {
    if (!plan_ok(p) || !Bir || !Bic) return (int)cudaErrorInvalidValue;
    if (ncols != p->ncols || nnz != p->nnz) return (int)cudaErrorInvalidValue;
    cudaStream_t st = as_stream(stream);
    cudaError_t err = cudaMemsetAsync(p->mismatch, 0, sizeof(int), st);
    if (err != cudaSuccess) return (int)err;
    plan_verify_kernel<<<148 * 16, 256, 0, st>>>((long long)nnz, p->perm, p->keys, p->cols, p->lay.rowmask, Bir, Bic,
                                                 p->mismatch);
    g_launches += 1;
    int h = 0;
    err = cudaMemcpyAsync(&h, p->mismatch, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (err == cudaSuccess) err = cudaStreamSynchronize(st);
    if (err != cudaSuccess) return (int)err;
    return h ? (int)cudaErrorInvalidValue : 0;
}

int bidmat_b200_plan_info(bidmat_b200_plan_t p, long long *out, int count) {
    if (!p || p->magic != kPlanMagic || !out || count < 0) return (int)cudaErrorInvalidValue;
    const long long v[BIDMAT_B200_PLAN_INFO_COUNT] = {
        p->nnz, p->ncols, p->m, p->k, p->elem, p->lay.nblocks, p->nchunks, p->nruns, p->nslots,
        p->nclear, p->touched_rows, (long long)p->bytes, p->row_runs};
    for (int i = 0; i < count && i < BIDMAT_B200_PLAN_INFO_COUNT; i++) out[i] = v[i];
    return 0;
}

int bidmat_b200_plan_touched_rows(bidmat_b200_plan_t p, unsigned *bitmap, bidmat_stream_t stream) {
    if (!plan_ok(p) || !bitmap) return (int)cudaErrorInvalidValue;
    return (int)cudaMemcpyAsync(bitmap, p->touched, (((size_t)p->m + 31) / 32) * sizeof(unsigned),
                                cudaMemcpyDeviceToDevice, as_stream(stream));
}

int bidmat_b200_plan_clear_untouched(bidmat_b200_plan_t p, int nrows, void *C, bidmat_stream_t stream) {
    if (!plan_ok(p) || !C || nrows != p->k) return (int)cudaErrorInvalidValue;
    cudaStream_t st = as_stream(stream);
    const unsigned blocks = (unsigned)(((size_t)p->m * 32 + 255) / 256);
    if (p->elem == 4) plan_clear_untouched_kernel<float><<<blocks, 256, 0, st>>>(p->k, p->m, p->touched, static_cast<float *>(C));
    else plan_clear_untouched_kernel<double><<<blocks, 256, 0, st>>>(p->k, p->m, p->touched, static_cast<double *>(C));
    g_launches += 1;
    return (int)cudaGetLastError();
}

int bidmat_b200_plan_destroy(bidmat_b200_plan_t p) {
    if (!p) return 0;
    if (p->magic != kPlanMagic) return (int)cudaErrorInvalidValue;
    const int dev = p->dev;
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    cudaError_t err = cudaDeviceSynchronize();     // a call using the plan may still be in flight
    plan_free(p);
    if (prev >= 0 && prev != dev) cudaSetDevice(prev);
    return (int)err;
}

}  // extern "C"
