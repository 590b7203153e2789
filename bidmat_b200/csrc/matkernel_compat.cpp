// The launcher symbols of BIDMat's jni/include/MatKernel.hpp (and the double
// overloads of MatKernelD.hpp) for the sparse-dense path, implemented on this
// library's C ABI.  Linked into BIDMat's libbidmatcuda in place of the same
// functions of jni/src/Arith.cu, jni/src/Operators.cu and jni/src/MatKernelD.cu,
// it lets the reference's own JNI glue (jni/src/BIDMat_CUMAT.cpp:252-293, 722-798,
// 873-881, 1456-1471; BIDMat_CUMATD.cpp) link unchanged: same C++ names, same
// argument lists, same return convention (a cudaError_t as int after a
// synchronisation of the per-thread default stream).
//
// This file is NOT part of libbidmatcuda_b200.so: a process that also loads the
// stock library would then hold two definitions of each name.  The build writes
// it as an object file (lib/matkernel_compat.o) to be linked on BIDMat's side
// together with -lbidmatcuda_b200.
#include "../../include/bidmat_b200.h"

// jni/include/MatKernel.hpp:140, jni/src/Arith.cu:46-60
int dsmult(int nrows, int ncols, int nnz, float *A, float *Bdata, int *Bir, int *Bic, float *C) {
    return bidmat_b200_dsmult(nrows, ncols, nnz, A, Bdata, Bir, Bic, C);
}

// jni/include/MatKernel.hpp:150, jni/src/Arith.cu:234-248
int dsmultT(int nrows, int ncols, int nnz, float *A, float *Bdata, int *Bir, int *Bic, float *C) {
    return bidmat_b200_dsmultT(nrows, ncols, nnz, A, Bdata, Bir, Bic, C);
}

// jni/include/MatKernel.hpp:154, jni/src/Arith.cu:381-389
int dds(int nrows, int nnz, float *A, float *B, int *Cir, int *Cic, float *P) {
    return bidmat_b200_dds(nrows, nnz, A, B, Cir, Cic, P);
}

// jni/include/MatKernel.hpp:156, jni/src/Arith.cu:391-399 (the last index array holds column pointers)
int dds0(int nrows, int ncols, float *A, float *B, int *Cir, int *Cjc, float *P) {
    return bidmat_b200_dds0(nrows, ncols, A, B, Cir, Cjc, P);
}

// jni/include/MatKernel.hpp:146,148, jni/src/Arith.cu:191-204: the launch shape is accepted and ignored
int dsmult_tune(int nrows, int ncols, int nnz, float *A, float *Bdata, int *Bir, int *Bic, float *C, int nblocks,
                int nthreads) {
    return bidmat_b200_dsmult_tune(nrows, ncols, nnz, A, Bdata, Bir, Bic, C, nblocks, nthreads);
}

int dsmultx_tune(int nrows, int ncols, int nnz, float *A, float *Bdata, int *Bir, int *Bic, float *C, int nblocks,
                 int nthreadsx, int nthreadsy) {
    return bidmat_b200_dsmultx_tune(nrows, ncols, nnz, A, Bdata, Bir, Bic, C, nblocks, nthreadsx, nthreadsy);
}

// jni/include/MatKernel.hpp:142,144, jni/src/Arith.cu:159-189
int dsmultTile(int nr, int nc, int kk, int nnz, float *A, int lda, float *Bdata, int *Bir, int *Bic, int broff,
               int bcoff, float *C, int ldc) {
    return bidmat_b200_dsmultTile(nr, nc, kk, nnz, A, lda, Bdata, Bir, Bic, broff, bcoff, C, ldc, 0);
}

int dsmultTileT(int nr, int nc, int kk, int nnz, float *A, int lda, float *Bdata, int *Bir, int *Bic, int broff,
                int bcoff, float *C, int ldc) {
    return bidmat_b200_dsmultTile(nr, nc, kk, nnz, A, lda, Bdata, Bir, Bic, broff, bcoff, C, ldc, 1);
}

// jni/include/MatKernel.hpp:152, jni/src/Arith.cu:267-277
int spsum(int nrows, int ncols, int nnz, int *Air, int *Aic, float *P, float *B, int n) {
    return bidmat_b200_spsum(nrows, ncols, nnz, Air, Aic, P, B, n);
}

// jni/include/MatKernel.hpp:47,51, jni/src/Operators.cu:586-644
int sdoprow(int nrows, int ncols, int nnz, float *A, int *Aic, float *B, int len, int opn) {
    return bidmat_b200_sdoprow(nrows, ncols, nnz, A, Aic, B, len, opn);
}

int sdopcol(int nrows, int ncols, int nnz, float *A, int *Air, float *B, int len, int opn) {
    return bidmat_b200_sdopcol(nrows, ncols, nnz, A, Air, B, len, opn);
}

// ---- double overloads: jni/include/MatKernelD.hpp:43,49,51,53,55 and MatKernel.hpp:49,53
int dsmult(int nrows, int ncols, int nnz, double *A, double *Bdata, int *Bir, int *Bic, double *C) {
    return bidmat_b200_dsmult_f64(nrows, ncols, nnz, A, Bdata, Bir, Bic, C);
}

int dsmultT(int nrows, int ncols, int nnz, double *A, double *Bdata, int *Bir, int *Bic, double *C) {
    return bidmat_b200_dsmultT_f64(nrows, ncols, nnz, A, Bdata, Bir, Bic, C);
}

int dds(int nrows, int nnz, double *A, double *B, int *Cir, int *Cic, double *P) {
    return bidmat_b200_dds_f64(nrows, nnz, A, B, Cir, Cic, P);
}

int dds0(int nrows, int ncols, double *A, double *B, int *Cir, int *Cjc, double *P) {
    return bidmat_b200_dds0_f64(nrows, ncols, A, B, Cir, Cjc, P);
}

int spsum(int nrows, int ncols, int nnz, int *Air, int *Aic, double *P, double *B, int n) {
    return bidmat_b200_spsum_f64(nrows, ncols, nnz, Air, Aic, P, B, n);
}

int sdoprow(int nrows, int ncols, int nnz, double *A, int *Aic, double *B, int len, int opn) {
    return bidmat_b200_sdoprow_f64(nrows, ncols, nnz, A, Aic, B, len, opn);
}

int sdopcol(int nrows, int ncols, int nnz, double *A, int *Air, double *B, int len, int opn) {
    return bidmat_b200_sdopcol_f64(nrows, ncols, nnz, A, Air, B, len, opn);
}
