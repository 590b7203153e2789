/*
 * bidmat_b200.h -- C ABI of the B200 (sm_100a) sparse-dense library.
 *
 * This is the drop-in boundary for BIDMat's native calls on one path: the
 * dense x sparse products behind GMat*GSMat and GMat*^GSMat and the sampled
 * dense-dense product DDS.  Every function takes plain device pointers and
 * sizes, returns a cudaError_t cast to int (0 = success) and never aborts the
 * process.  Conventions shared by all entry points:
 *
 *   - dense matrices are column-major fp32 with leading dimension nrows (k):
 *     column c starts at base + c*nrows  (BIDMat GMat.pdata layout,
 *     src/main/scala/BIDMat/GMat.scala:20);
 *   - a sparse matrix is BIDMat's GSMat device layout
 *     (src/main/scala/BIDMat/GSMat.scala:14-15): int32 0-based row index per
 *     nonzero (pir), int32 0-based column index per nonzero in non-decreasing
 *     order (pic), fp32 value per nonzero (pdata), and int32 column pointers
 *     (pjc, ncols+1 entries) where a function says so;
 *   - rows inside a column may be unsorted or repeated; empty columns are fine;
 *   - all pointers are owned by the caller and live on the calling thread's
 *     current device; only the output array is written;
 *   - nnz == 0 is a successful no-op.
 *
 * The four functions without suffix are synchronous on the per-thread default
 * stream, exactly like the launchers they replace.  The *_async variants
 * enqueue on a caller-supplied stream and return without synchronising.
 * Scratch memory, where an operation needs it, is allocated stream-ordered from a
 * per-device pool owned by the library and returned before the call ends (see
 * bidmat_b200_release_workspace / bidmat_b200_set_workspace_limit).
 */
#ifndef BIDMAT_B200_H
#define BIDMAT_B200_H

#if defined(__GNUC__)
#define BIDMAT_B200_API __attribute__((visibility("default")))
#else
#define BIDMAT_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque stream handle: a cudaStream_t passed as void* so that this header
 * needs no CUDA include. NULL selects the per-thread default stream. */
typedef void *bidmat_stream_t;

/* C(nrows x ncols) += A(nrows x m) * S(m x ncols).
 * Replaces: int dsmult(int,int,int,float*,float*,int*,int*,float*)
 *   jni/include/MatKernel.hpp:140, jni/src/Arith.cu:46-60, bound from
 *   CUMAT.dsmult (src/main/java/edu/berkeley/bid/CUMAT.java:143) through
 *   Java_edu_berkeley_bid_CUMAT_dsmult (jni/src/BIDMat_CUMAT.cpp:722-733). */
BIDMAT_B200_API int bidmat_b200_dsmult(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                       const int *Bir, const int *Bic, float *C);

/* C(nrows x m) += A(nrows x ncols) * S(m x ncols)^T.  m is not passed by the
 * reference interface; the rows written are exactly those named in Bir.
 * Replaces: int dsmultT(...) jni/include/MatKernel.hpp:150,
 *   jni/src/Arith.cu:234-248, CUMAT.dsmultT (CUMAT.java:152),
 *   Java_edu_berkeley_bid_CUMAT_dsmultT (BIDMat_CUMAT.cpp:761-772). */
BIDMAT_B200_API int bidmat_b200_dsmultT(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                        const int *Bir, const int *Bic, float *C);

/* P[j] += <A[:, Cir[j]], B[:, Cic[j]]> for j in [0, nnz).
 * Replaces: int dds(int,int,float*,float*,int*,int*,float*)
 *   jni/include/MatKernel.hpp:154, jni/src/Arith.cu:381-389, CUMAT.dds
 *   (CUMAT.java:211), Java_edu_berkeley_bid_CUMAT_dds
 *   (BIDMat_CUMAT.cpp:774-785). */
BIDMAT_B200_API int bidmat_b200_dds(int nrows, int nnz, const float *A, const float *B, const int *Cir,
                    const int *Cic, float *P);

/* P[j] = <A[:, Cir[j]], B[:, c]> for j in [Cjc[c], Cjc[c+1]), c in [0, ncols):
 * the column-pointer driven form, which stores instead of accumulating.
 * Valid for any nrows (the reference kernel is only meaningful for 1024).
 * Replaces: int dds0(int,int,float*,float*,int*,int*,float*)
 *   jni/include/MatKernel.hpp:156, jni/src/Arith.cu:391-399, CUMAT.dds0
 *   (CUMAT.java:213), Java_edu_berkeley_bid_CUMAT_dds0
 *   (BIDMat_CUMAT.cpp:787-798). */
BIDMAT_B200_API int bidmat_b200_dds0(int nrows, int ncols, const float *A, const float *B, const int *Cir,
                     const int *Cjc, float *P);

/* Launch-shape tuning hooks of the reference: same result as dsmult; the
 * shape arguments are accepted and ignored.
 * Replaces: dsmult_tune / dsmultx_tune (jni/include/MatKernel.hpp:146-148,
 *   jni/src/Arith.cu:191-204, CUMAT.java:148-150, BIDMat_CUMAT.cpp:735-759). */
BIDMAT_B200_API int bidmat_b200_dsmult_tune(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                            const int *Bir, const int *Bic, float *C, int nblocks, int nthreads);
BIDMAT_B200_API int bidmat_b200_dsmultx_tune(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                             const int *Bir, const int *Bic, float *C, int nblocks, int nthreadsx,
                             int nthreadsy);

/* Stream-ordered forms of the four operations.  They enqueue on `stream` and do
 * not wait for the result.  dsmultT_async takes the row count m of S (it must
 * exceed every row index in Bir; <= 0 when unknown: the library then finds the
 * largest row index itself, which costs a host round trip inside the call).  When
 * the dense operand of dsmultT is much larger than the L2 cache the nonzeros are
 * processed in column blocks and the call waits once, internally, for the block
 * boundaries (a few bytes) before it enqueues the rest. */
BIDMAT_B200_API int bidmat_b200_dsmult_async(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                             const int *Bir, const int *Bic, float *C, bidmat_stream_t stream);
BIDMAT_B200_API int bidmat_b200_dsmultT_async(int nrows, int ncols, int nnz, const float *A, const float *Bdata,
                              const int *Bir, const int *Bic, float *C, int m_hint,
                              bidmat_stream_t stream);
BIDMAT_B200_API int bidmat_b200_dds_async(int nrows, int nnz, const float *A, const float *B, const int *Cir,
                          const int *Cic, float *P, bidmat_stream_t stream);
BIDMAT_B200_API int bidmat_b200_dds0_async(int nrows, int ncols, int nnz, const float *A, const float *B,
                           const int *Cir, const int *Cjc, float *P, bidmat_stream_t stream);

/* A*S and DDS(A,B,S) on the same sparse matrix in one pass:
 *     C(nrows x ncols) += A(nrows x m) * S          and          P[j] += <A[:, Sir[j]], B[:, Sic[j]]>
 * with S = (Sdata, Sir, Sic).  Same results as bidmat_b200_dsmult_async followed by
 * bidmat_b200_dds_async (each output is computed by the same arithmetic as in the separate
 * kernels).  Both operations gather the same column of A for every nonzero and that gather bounds
 * either of them; for fp32 operands with nrows in {128, 256, 512} and 16-byte aligned pointers one
 * kernel does it once for both, other shapes run the two operations one after the other.
 * Stream-ordered.  No counterpart in the reference's native interface: there the two are separate
 * calls (CUMAT.dsmult, CUMAT.dds: CUMAT.java:143,211), made one after the other on the same
 * operands by factorisation loops (P = DDS(A,B,S); C = A*S). */
BIDMAT_B200_API int bidmat_b200_dsmult_dds_async(int nrows, int ncols, int nnz, const float *A, const float *B,
                                                 const float *Sdata, const int *Sir, const int *Sic, float *C,
                                                 float *P, bidmat_stream_t stream);

/* Double-precision twins of the four operations (BIDMat's GDMat / GSDMat path).
 * Same semantics as the fp32 functions above; dense operands and values are fp64.
 * Replaces: dsmult / dsmultT / dds / dds0 on doubles (jni/include/MatKernelD.hpp:43,49,53,55,
 *   jni/src/MatKernelD.cu:780-1030, CUMATD.java:51,57,89,91). */
BIDMAT_B200_API int bidmat_b200_dsmult_f64(int nrows, int ncols, int nnz, const double *A, const double *Bdata,
                                           const int *Bir, const int *Bic, double *C);
BIDMAT_B200_API int bidmat_b200_dsmultT_f64(int nrows, int ncols, int nnz, const double *A, const double *Bdata,
                                            const int *Bir, const int *Bic, double *C);
BIDMAT_B200_API int bidmat_b200_dds_f64(int nrows, int nnz, const double *A, const double *B, const int *Cir,
                                        const int *Cic, double *P);
BIDMAT_B200_API int bidmat_b200_dds0_f64(int nrows, int ncols, const double *A, const double *B, const int *Cir,
                                         const int *Cjc, double *P);
BIDMAT_B200_API int bidmat_b200_dsmult_f64_async(int nrows, int ncols, int nnz, const double *A,
                                                 const double *Bdata, const int *Bir, const int *Bic,
                                                 double *C, bidmat_stream_t stream);
BIDMAT_B200_API int bidmat_b200_dsmultT_f64_async(int nrows, int ncols, int nnz, const double *A,
                                                  const double *Bdata, const int *Bir, const int *Bic,
                                                  double *C, int m_hint, bidmat_stream_t stream);
BIDMAT_B200_API int bidmat_b200_dds_f64_async(int nrows, int nnz, const double *A, const double *B,
                                              const int *Cir, const int *Cic, double *P,
                                              bidmat_stream_t stream);

/* Prepared transposed product.  bidmat_b200_dsmultT has to sort the nonzeros by row on
 * every call, because the reference interface hands it nothing but raw arrays.  A caller
 * that multiplies with the same sparse STRUCTURE again and again (any values) can prepare
 * it once:
 *   plan_create  sorts (Bir, Bic) of an m x ncols matrix for dense operands of `nrows`
 *                rows of elem_bytes (4 or 8) each and keeps the sorted list, the source
 *                position of every nonzero and the chunk layout on the device
 *                (about 12 bytes per nonzero, freed by plan_destroy).  Synchronous.
 *   planned      C(nrows x m) += A(nrows x ncols) * S^T with S = (Bir, Bic, Bdata): only
 *                the values are read through the stored positions; no sort, no host round
 *                trip, stream-ordered.  nrows, ncols and nnz must be those of the plan
 *                (cudaErrorInvalidValue otherwise).  With BIDMAT_B200_PLAN_OVERWRITE the
 *                columns of C named by at least one nonzero are overwritten with the
 *                product instead of added to, and all other columns are left untouched
 *                (plan_touched_rows tells which): a caller that would clear C first saves
 *                the clearing and one read of C.
 *   plan_verify  exact check that (Bir, Bic) is the structure the plan was made from
 *                (0 = yes, cudaErrorInvalidValue = no).  Synchronous.
 * A plan belongs to the device it was created on and may be used by one call at a time
 * (calls on one stream, or ordered by the caller).  The result is bit-reproducible and
 * uses no float atomics; terms of one output column are added in ascending source column
 * inside a column block, blocks in ascending order, pieces of rows split over chunks last.
 * No counterpart in the reference's native interface; the precedent is structure derived
 * once and kept on the matrix object (GSMat.fromSMat computing pic,
 * src/main/scala/BIDMat/GSMat.scala:620-647; DDS copying its argument's pattern,
 * GSMat.scala:656-661).  Replaces the per-call work of dsmultT (jni/src/Arith.cu:234-248). */
typedef struct bidmat_b200_plan *bidmat_b200_plan_t;
#define BIDMAT_B200_PLAN_OVERWRITE 1
BIDMAT_B200_API int bidmat_b200_dsmultT_plan_create(int nrows, int ncols, int nnz, int m, const int *Bir,
                                                    const int *Bic, int elem_bytes, bidmat_stream_t stream,
                                                    bidmat_b200_plan_t *plan);
BIDMAT_B200_API int bidmat_b200_dsmultT_planned(bidmat_b200_plan_t plan, int nrows, int ncols, int nnz,
                                                const float *A, const float *Bdata, float *C, int flags,
                                                bidmat_stream_t stream);
BIDMAT_B200_API int bidmat_b200_dsmultT_planned_f64(bidmat_b200_plan_t plan, int nrows, int ncols, int nnz,
                                                    const double *A, const double *Bdata, double *C, int flags,
                                                    bidmat_stream_t stream);
BIDMAT_B200_API int bidmat_b200_plan_verify(bidmat_b200_plan_t plan, int ncols, int nnz, const int *Bir,
                                            const int *Bic, bidmat_stream_t stream);
/* out[0..count): nnz, ncols, m, nrows, elem_bytes, column blocks, chunks, split runs, slots,
 * rows cleared by an overwriting call, rows named by at least one nonzero, device bytes held,
 * (column block, row) runs (each updates its output column once per call). */
#define BIDMAT_B200_PLAN_INFO_COUNT 13
BIDMAT_B200_API int bidmat_b200_plan_info(bidmat_b200_plan_t plan, long long *out, int count);
/* Copies to the device array `bitmap` (ceil(m/32) words, caller-owned) which rows of S hold a
 * nonzero: bit r%32 of word r/32 is set for such a row r.  Stream-ordered. */
BIDMAT_B200_API int bidmat_b200_plan_touched_rows(bidmat_b200_plan_t plan, unsigned *bitmap,
                                                  bidmat_stream_t stream);
/* A plan with a single column block (the dense operand fits the L2 rule: small problems, or one
 * rank's shard on many GPUs) can be run in `nparts` consecutive ROW RANGES of the result:
 * plan_row_parts fixes the ranges (row_bounds[0..nparts], ascending, 0 and m at the ends) and
 * planned_part computes the columns of C in range `part` completely (its chunks, then the fix-up of
 * the split rows inside it, with BIDMAT_B200_PLAN_OVERWRITE the clearing of its never-stored rows).
 * Calling every part once, in any order, on one stream gives what bidmat_b200_dsmultT_planned gives;
 * a consumer of finished rows (the sum over the ranks) can start while the other parts still run.  cudaErrorNotSupported (801): several column blocks, a
 * shape other than fp32 with nrows in {32 .. 512} and aligned pointers, or fewer chunks than parts. */
BIDMAT_B200_API int bidmat_b200_plan_row_parts(bidmat_b200_plan_t plan, int nparts, int *row_bounds);
BIDMAT_B200_API int bidmat_b200_dsmultT_planned_part(bidmat_b200_plan_t plan, int nrows, int ncols, int nnz,
                                                     const float *A, const float *Bdata, float *C, int flags,
                                                     int part, bidmat_stream_t stream);

/* Zeroes the columns of C (nrows x m, of the plan's element type) that no nonzero of S names: with
 * BIDMAT_B200_PLAN_OVERWRITE before it, C then equals the product everywhere without a full clear
 * (what a sum over whole buffers, e.g. bidmat_b200_mc_allreduce_sum, needs).  Stream-ordered. */
BIDMAT_B200_API int bidmat_b200_plan_clear_untouched(bidmat_b200_plan_t plan, int nrows, void *C,
                                                     bidmat_stream_t stream);
BIDMAT_B200_API int bidmat_b200_plan_destroy(bidmat_b200_plan_t plan);

/* Plans kept by the library, for a binding that cannot hold a handle (the natives of CUMAT.java:152
 * rebound as they are).  With set_auto_plan(1), or BIDMAT_B200_AUTO_PLAN=1 in the environment, the
 * SYNCHRONOUS entry points bidmat_b200_dsmultT and bidmat_b200_dsmultT_f64 take a 128-bit
 * fingerprint of (Bir, Bic) on every call (one coalesced pass over the two arrays and a 24-byte
 * read-back), build a plan for a structure when they see it for the second time, and run every later
 * call whose nrows, ncols, nnz, element type and fingerprint match through it, accumulating like the
 * ordinary path (same tolerance; the order of the additions is the plan's).  At most 2 plans are kept
 * per GPU (least recently used goes first); a structure seen only once costs no plan.  Pointers are
 * never part of the key.  Off by default: a kept plan holds about 13 bytes per nonzero of device
 * memory.  set_auto_plan(0) switches it off and frees the kept plans.
 * auto_plan_info fills out[0..count): enabled, plans built, calls that ran through a plan, calls that
 * took the ordinary path while it was on, plans kept now, device bytes they hold. */
BIDMAT_B200_API int bidmat_b200_set_auto_plan(int enable);
BIDMAT_B200_API int bidmat_b200_auto_plan_info(long long *out, int count);

/* A*S without any allocation.  No counterpart in the reference: BIDMat's
 * launchers never needed scratch memory.  It exists for callers that cannot let a
 * library allocate on the device: host applications that have handed all device
 * memory to their own caching allocator (BIDMat's GPU cache, a full PyTorch pool),
 * where a cudaMalloc from inside this library may fail or fragment that pool, and
 * multi-stream serving loops that cannot afford the device-wide synchronisation
 * cudaMalloc/cudaFree imply.
 *
 * Same result and same stream-ordered behaviour as bidmat_b200_dsmult_async (the
 * sums of columns split over different chunk boundaries may differ in the last
 * bits).  The scratch is a fixed array of BIDMAT_B200_NOALLOC_SCRATCH_FLOATS
 * floats (16 MiB) that every GPU loading the library holds until exit.
 *   Limit: 2*nrows*ceil(nnz/chunk) floats must fit the array for some chunk
 *   length <= BIDMAT_B200_NOALLOC_MAX_CHUNK, i.e.
 *       nnz <= BIDMAT_B200_NOALLOC_MAX_CHUNK * floor(SCRATCH_FLOATS / (2*nrows))
 *   (134,217,728 nonzeros at nrows = 256).  Larger problems are rejected with
 *   cudaErrorInvalidValue before anything is launched; use dsmult_async then.
 *   First call on a device: resolves the array's device address with
 *   cudaGetSymbolAddress.  Make that first call outside any stream capture.
 *   Sharing: all calls on a device use the same array and it keeps the previous
 *   call's contents (nothing needs clearing: every slot read is written earlier
 *   in the same call).  Calls that overlap on the GPU race on it; keep them on
 *   one stream or order them with events. */
#define BIDMAT_B200_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define BIDMAT_B200_NOALLOC_MAX_CHUNK 16384
BIDMAT_B200_API int bidmat_b200_dsmult_noalloc(int nrows, int ncols, int nnz, const float *A,
                                               const float *Bdata, const int *Bir, const int *Bic,
                                               float *C, bidmat_stream_t stream);

/* Sum over the GPUs of one box of the per-GPU partial results of B*^S, through
 * NVLink peer memory instead of a communication library.  peer_addresses[r] is the
 * device address, valid on the calling GPU, of rank r's buffer of `count` floats
 * (16-byte aligned, count a multiple of 4; world is 2, 4 or 8).  The calling rank
 * sums its 1/world slice of all buffers in rank order with peer loads and writes the
 * total into all buffers with peer stores, so all GPUs end with bit-identical
 * results.  Stream-ordered on `stream` with `ctas` CTAs of 256 threads (<= 0: 64 / 48 / 32
 * for 2 / 4 / 8 GPUs).
 * The kernel never waits on another GPU: the caller synchronises the ranks before
 * (all partials complete) and after (all slices written).
 * Replaces the role of NCCL.ncclAllReduce in GFunctions.ncclAllReduce
 *   (src/main/scala/BIDMat/GFunctions.scala:175-203, jni/src/BIDMat_NCCL.cpp:80-90). */
BIDMAT_B200_API int bidmat_b200_peer_allreduce_sum(int world, int rank, const unsigned long long *peer_addresses,
                                                   long long count, int ctas, bidmat_stream_t stream);

/* The same sum for a k x m result (k % 4 == 0) when it is known which of its m columns
 * ("rows" of the sparse matrix) every rank wrote: touched is a device array of
 * world * ceil(m/32) words, rank r's bitmap first to last (bidmat_b200_plan_touched_rows of
 * each rank's plan, gathered once).  A rank's column is read only when that rank wrote it,
 * so no rank has to clear its buffer between steps (columns it did not write may hold the
 * previous sum) and less crosses NVLink; columns nobody wrote are set to zero.  Together
 * with BIDMAT_B200_PLAN_OVERWRITE this removes the clearing of the k x m partial from the
 * step.  ctas <= 0: 64 CTAs for 2 GPUs, 48 for 4 or 8.  Same ordering rules as
 * bidmat_b200_peer_allreduce_sum. */
BIDMAT_B200_API int bidmat_b200_peer_allreduce_sum_rows(int world, int rank,
                                                        const unsigned long long *peer_addresses, int k,
                                                        long long m, const unsigned *touched, int ctas,
                                                        bidmat_stream_t stream);
/* The same for the columns [row_begin, row_end) only (a row range of a plan run in parts). */
BIDMAT_B200_API int bidmat_b200_peer_allreduce_sum_rows_range(int world, int rank,
                                                              const unsigned long long *peer_addresses, int k,
                                                              long long m, const unsigned *touched,
                                                              long long row_begin, long long row_end, int ctas,
                                                              bidmat_stream_t stream);

/* The same sum through the NVSwitch, for buffers that are bound to a multicast object:
 * multicast_address is the multicast mapping of the ranks' buffers of `count` floats (count a
 * multiple of 4).  The calling rank reduces its 1/world slice with multimem.ld_reduce (the switch
 * fetches it from every GPU and adds on the way) and stores the total into all buffers with
 * multimem.st, so about half as many bytes cross NVLink per GPU and direction as with peer loads
 * and stores, and all ranks end bit-identical (the order of the additions is the switch's).
 * Whole buffers are summed: rows a rank did not write must hold zeros
 * (bidmat_b200_plan_clear_untouched).  ctas <= 0: 96 CTAs on 8 GPUs, 64 otherwise.  Same ordering
 * rules as bidmat_b200_peer_allreduce_sum. */
BIDMAT_B200_API int bidmat_b200_mc_allreduce_sum(int world, int rank, void *multicast_address, long long count,
                                                 int ctas, bidmat_stream_t stream);
/* The same over the floats [first, first + count) of the buffers only (both multiples of 4): the rows
 * of a row range of a prepared product (bidmat_b200_dsmultT_planned_part) once every rank has computed them. */
BIDMAT_B200_API int bidmat_b200_mc_allreduce_sum_range(int world, int rank, void *multicast_address, long long first,
                                                       long long count, int ctas, bidmat_stream_t stream);

/* Structure helpers on the device (the steps BIDMat performs around the path
 * with cuSPARSE csr2coo and a host loop: GSMat.fromSMat, GSMat.scala:639, and
 * SparseMat.compressInds, SparseMat.scala:857-868).
 *   expand:   ic[j] = c for j in [jc[c], jc[c+1])
 *   compress: jc[c] = number of nonzeros with ic < c, c in [0, ncols] */
BIDMAT_B200_API int bidmat_b200_expand_jc(int ncols, int nnz, const int *jc, int *ic, bidmat_stream_t stream);
BIDMAT_B200_API int bidmat_b200_compress_ic(int ncols, int nnz, const int *ic, int *jc, bidmat_stream_t stream);

/* Transpose of a GSMat on the device: T = S^T, S is nrows x ncols.  Inputs are S's
 * per-nonzero rows, per-nonzero columns (non-decreasing) and values; outputs are
 * T's per-nonzero rows (t_ir = S's columns), per-nonzero columns (t_ic = S's rows,
 * non-decreasing), values, and optionally T's column pointers t_jc (nrows+1
 * entries, may be NULL).  Rows come out ascending inside every column of T.
 * Replaces the host round trip of GSMat.t (src/main/scala/BIDMat/GSMat.scala:218-223:
 * download, SMat.t on the CPU, upload).  Stream-ordered, uses the workspace. */
BIDMAT_B200_API int bidmat_b200_transpose_csc(int nrows, int ncols, int nnz, const int *ir, const int *ic,
                                              const float *data, int *t_ir, int *t_ic, int *t_jc,
                                              float *t_data, bidmat_stream_t stream);

/* Tiled products for BIDMat's TMat.  A is an nr x kk tile (leading dimension lda) of a
 * dense matrix and C an nr x nc tile (leading dimension ldc); only the nonzeros of S
 * inside the tile take part, with indices taken relative to (broff, bcoff):
 *   transpose == 0: rows [broff, broff+kk), columns [bcoff, bcoff+nc):
 *                   C[:, col-bcoff] += A[:, row-broff] * value
 *   transpose != 0: rows [broff, broff+nc), columns [bcoff, bcoff+kk):
 *                   C[:, row-broff] += A[:, col-bcoff] * value
 * Accumulates without float atomics.  Synchronous.
 * Replaces: dsmultTile / dsmultTileT (jni/include/MatKernel.hpp:142-144,
 *   jni/src/Arith.cu:63-189, CUMAT.dsmultTile CUMAT.java:145-146,
 *   Java_edu_berkeley_bid_CUMAT_dsmultTile BIDMat_CUMAT.cpp:1456-1471). */
BIDMAT_B200_API int bidmat_b200_dsmultTile(int nr, int nc, int kk, int nnz, const float *A, int lda,
                                           const float *Bdata, const int *Bir, const int *Bic, int broff,
                                           int bcoff, float *C, int ldc, int transpose);

/* Edge operators on the values of a GSMat: A[j] = op(A[j], B[Aic[j]]) (sdoprow, B is
 * a 1 x ncols row) or op(A[j], B[Air[j]]) (sdopcol, B is an nrows x 1 column); with
 * len == 1 every value is combined with B[0].  opn indexes BIDMat's operator table
 * (0 add, 1 sub, 2 mul, 3 div, 4 gt, 5 lt, 6 eq, 7 ge, 8 le, 9 ne, 10 max, 11 min,
 * 12 atan2, 13 pow, 14 ifpos; jni/src/Operators.cu:86-101).  Synchronous.
 * Replaces: sdoprow / sdopcol (jni/include/MatKernel.hpp:47,51,
 *   jni/src/Operators.cu:586-644, CUMAT.java:135,139, BIDMat_CUMAT.cpp:252-293). */
BIDMAT_B200_API int bidmat_b200_sdoprow(int nrows, int ncols, int nnz, float *A, const int *Aic, const float *B,
                                        int len, int opn);
BIDMAT_B200_API int bidmat_b200_sdopcol(int nrows, int ncols, int nnz, float *A, const int *Air, const float *B,
                                        int len, int opn);
/* Double-precision edge operators: BIDMat binds them as separate natives, sdopdrow / sdopdcol
 * (CUMAT.java:137,141, BIDMat_CUMAT.cpp:263-271, 284-293), onto the double overloads of
 * sdoprow / sdopcol (jni/include/MatKernel.hpp:49,53). */
BIDMAT_B200_API int bidmat_b200_sdoprow_f64(int nrows, int ncols, int nnz, double *A, const int *Aic,
                                            const double *B, int len, int opn);
BIDMAT_B200_API int bidmat_b200_sdopcol_f64(int nrows, int ncols, int nnz, double *A, const int *Air,
                                            const double *B, int len, int opn);

/* Sums of the values of a GSMat: n == 1: B(1 x ncols)[Aic[j]] += P[j] (column sums);
 * otherwise B(nrows x 1)[Air[j]] += P[j] (row sums).  Accumulates, without float
 * atomics (the reference adds with atomicAdd), so the result is bit-reproducible.
 * Synchronous.
 * Replaces: spsum (jni/include/MatKernel.hpp:152, jni/src/Arith.cu:250-277,
 *   CUMAT.java:209, BIDMat_CUMAT.cpp:873-881). */
BIDMAT_B200_API int bidmat_b200_spsum(int nrows, int ncols, int nnz, const int *Air, const int *Aic,
                                      const float *P, float *B, int n);
/* Double-precision twin (spsum on doubles, jni/include/MatKernelD.hpp:51, CUMATD.java:71). */
BIDMAT_B200_API int bidmat_b200_spsum_f64(int nrows, int ncols, int nnz, const int *Air, const int *Aic,
                                          const double *P, double *B, int n);

/* Validates a GSMat structure on the device without touching values:
 * 0 <= ir < m, 0 <= ic < ncols, ic non-decreasing.  Returns 0 when it holds,
 * cudaErrorInvalidValue (1) when it does not, another cudaError_t on failure.
 * Synchronous. */
BIDMAT_B200_API int bidmat_b200_check_structure(int m, int ncols, int nnz, const int *ir, const int *ic);

/* Scratch memory.  Every call that needs scratch takes it from a memory pool the library
 * owns on the calling thread's device, by stream-ordered allocation on the call's stream,
 * and gives it back on that stream before returning; freed blocks stay cached in the pool
 * for the next call.  workspace_bytes: bytes the pool currently holds.  release_workspace:
 * hands everything that is not in use back to the driver.  set_workspace_limit: the largest
 * scratch request (bytes, 0 = unlimited) a single call may make on this device; a call that
 * needs more returns cudaErrorMemoryAllocation before launching anything and leaves the
 * device and the library usable (a host whose own allocator owns the device memory can
 * bound what this library takes). */
BIDMAT_B200_API long long bidmat_b200_workspace_bytes(void);
BIDMAT_B200_API int bidmat_b200_release_workspace(void);
BIDMAT_B200_API int bidmat_b200_set_workspace_limit(long long bytes);

/* Number of kernels this library has launched in this process (all devices);
 * the benchmark reports the difference across its timed region. */
BIDMAT_B200_API long long bidmat_b200_launch_count(void);

/* Optional per-kernel timing for benchmarks.  While enabled, the launchers
 * bracket their main kernels with CUDA events on the launching stream.
 * timing_read sums the spans recorded under `label` ("dsmult_ga_chunk",
 * "dsmultT_ga_chunk", "dsmultT_rowsort", "ga_fixup", "dds_chunk") after waiting
 * for them; timing_reset discards all spans.  All spans must belong to the
 * calling thread's current device. */
BIDMAT_B200_API int bidmat_b200_timing_enable(int on);
BIDMAT_B200_API int bidmat_b200_timing_read(const char *label, double *total_ms, long long *count);
BIDMAT_B200_API int bidmat_b200_timing_reset(void);

/* Library version, and the text of a cudaError_t for error messages. */
BIDMAT_B200_API int bidmat_b200_version(void);
BIDMAT_B200_API const char *bidmat_b200_error_string(int err);

#ifdef __cplusplus
}
#endif
#endif /* BIDMAT_B200_H */
