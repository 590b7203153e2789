/*
 * TEST INFRASTRUCTURE.  C entry points over the reference's own CUDA launchers
 * for the sparse-dense path.  oracle/build.py compiles this file together with
 * jni/src/Arith.cu taken from the reference tree where it lies (never copied)
 * into oracle/_ref/libarith_ref.so, for sm_100a, with refshim/legacy_shuffle.h
 * force-included.  Used by the GPU tests as a second checker (the reference's
 * GPU results on the same inputs) and by the benchmark to time the reference's
 * kernels beside this library's.  The launchers synchronise the legacy default
 * stream themselves and return a cudaError_t.
 *
 *   ref_gpu_dsmult   -> dsmult   jni/src/Arith.cu:46-60   (kernels :16-44)
 *   ref_gpu_dsmultT  -> dsmultT  jni/src/Arith.cu:234-248 (kernels :206-232)
 *   ref_gpu_dds      -> dds      jni/src/Arith.cu:381-389 (kernel  :291-310)
 *   ref_gpu_dds0     -> dds0     jni/src/Arith.cu:391-399 (kernel  :312-349;
 *                                 reads B[tid + k*col] for tid < 1024 whatever k
 *                                 is, so it may only be called with nrows == 1024)
 *   ref_gpu_spsum    -> spsum    jni/src/Arith.cu:267-277
 */
#include <MatKernel.hpp>

extern "C" {

int ref_gpu_dsmult(int nrows, int ncols, int nnz, float *A, float *Bdata, int *Bir, int *Bic, float *C) {
    return dsmult(nrows, ncols, nnz, A, Bdata, Bir, Bic, C);
}

int ref_gpu_dsmultT(int nrows, int ncols, int nnz, float *A, float *Bdata, int *Bir, int *Bic, float *C) {
    return dsmultT(nrows, ncols, nnz, A, Bdata, Bir, Bic, C);
}

int ref_gpu_dds(int nrows, int nnz, float *A, float *B, int *Cir, int *Cic, float *P) {
    return dds(nrows, nnz, A, B, Cir, Cic, P);
}

int ref_gpu_dds0(int nrows, int ncols, float *A, float *B, int *Cir, int *Cjc, float *P) {
    if (nrows != 1024) return 1;   /* cudaErrorInvalidValue: the reference kernel is only defined for 1024 rows */
    return dds0(nrows, ncols, A, B, Cir, Cjc, P);
}

int ref_gpu_spsum(int nrows, int ncols, int nnz, int *Air, int *Aic, float *P, float *B, int n) {
    return spsum(nrows, ncols, nnz, Air, Aic, P, B, n);
}

}  /* extern "C" */
