/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of BIDMat's own CPU path for the three sparse-dense
 * operations that the CUDA library accelerates.  Only the test-suite, the smoke
 * check and the CPU-baseline leg of the benchmark may load this file; the
 * product never calls it.
 *
 * Parity status:
 *   A*S   (oracle_dsmult)   pinned: bit-identical to the reference's own C loop
 *                           smcscm (jni/src/BIDMat_SPBLAS.c:364-395) compiled
 *                           from the reference tree (see oracle/build.py).
 *   B*^S  (oracle_dsmultT)  pinned: bit-identical to smcsrm
 *                           (jni/src/BIDMat_SPBLAS.c:397-427), same recipe.
 *   DDS   (oracle_dds)      arithmetic pinned: bit-identical to smcscm called
 *                           with a one-row dense operand, which adds v[j]*a[ir[j]]
 *                           in j order from a stored 0
 *                           (jni/src/BIDMat_SPBLAS.c:376-388), i.e. the
 *                           "dsum += a(k)*b(k)" loop of DDShelper
 *                           (src/main/scala/BIDMat/MatFunctions.scala:1603-1607);
 *                           stored as tests/golden/dds_ref_vectors.npz.  Which
 *                           (row, column) pair a nonzero samples is pinned by the
 *                           Scala source (MatFunctions.scala:1594-1618) and, in
 *                           the GPU tests, by the reference's own CUDA dds
 *                           (jni/src/Arith.cu:291-310, 381-389) compiled for
 *                           sm_100a; the reference has no test of DDS.
 *
 * All dense matrices are column-major fp32 with leading dimension k; S is CSC
 * with 0-based int32 jc[n+1], ir[nnz] and fp32 data[nnz].  Arithmetic is strict
 * fp32: one rounded multiply then one rounded add per term, accumulated directly
 * in the fp32 output, in exactly the order of the reference loops (the JVM
 * never contracts a*b+c).  Compile with -ffp-contract=off.
 */
#include <stdint.h>
#include <stddef.h>
#include <omp.h>

/* FMat.fSMultHelper, src/main/scala/BIDMat/FMat.scala:1112-1132:
 * for each column i (ascending), for j in [jc[i], jc[i+1]) ascending,
 *   out[:, i] += A[:, ir[j]] * data[j], elementwise with kk ascending.
 * Threading follows FMat.madd (FMat.scala:1174-1184): thread t owns the
 * contiguous column range [t*n/T, (t+1)*n/T). */
void oracle_dsmult(int k, int n, const float *A, const float *data, const int32_t *ir,
                   const int32_t *jc, float *C, int nthreads) {
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for num_threads(nthreads) schedule(static, 1)
    for (int t = 0; t < nthreads; t++) {
        int istart = (int)((int64_t)t * n / nthreads);
        int iend = (int)((int64_t)(t + 1) * n / nthreads);
        for (int i = istart; i < iend; i++) {
            float *out = C + (size_t)i * k;
            for (int j = jc[i]; j < jc[i + 1]; j++) {
                float dval = data[j];
                const float *a = A + (size_t)ir[j] * k;
                for (int kk = 0; kk < k; kk++) {
                    float prod = a[kk] * dval;
                    out[kk] = out[kk] + prod;
                }
            }
        }
    }
}

/* FMat.fSMultTHelper2, src/main/scala/BIDMat/FMat.scala:1369-1389:
 * for each column i (ascending), j ascending:
 *   out[kstart:kend, ir[j]] += B[kstart:kend, i] * data[j].
 * Threading follows FMat.maddT (FMat.scala:1415-1426): min(T, k/32) threads,
 * thread t owns rows [k*t/T', k*(t+1)/T') of the dense matrices and scans ALL of
 * S; below 64 rows a single thread does everything. */
void oracle_dsmultT(int k, int n, const float *B, const float *data, const int32_t *ir,
                    const int32_t *jc, float *C, int nthreads) {
    int nt = 1;
    if (k >= 64 && nthreads > 1) {
        nt = nthreads < k / 32 ? nthreads : k / 32;
        if (nt < 1) nt = 1;
    }
#pragma omp parallel for num_threads(nt) schedule(static, 1)
    for (int t = 0; t < nt; t++) {
        int kstart = (int)((int64_t)k * t / nt);
        int kend = (int)((int64_t)k * (t + 1) / nt);
        for (int i = 0; i < n; i++) {
            const float *b = B + (size_t)i * k;
            for (int j = jc[i]; j < jc[i + 1]; j++) {
                float dval = data[j];
                float *out = C + (size_t)ir[j] * k;
                for (int kk = kstart; kk < kend; kk++) {
                    float prod = b[kk] * dval;
                    out[kk] = out[kk] + prod;
                }
            }
        }
    }
}

/* MatFunctions.DDShelper, src/main/scala/BIDMat/MatFunctions.scala:1594-1618:
 * P.data[j] = sum_kk A[kk, ir[j]] * B[kk, i] for j in column i, fp32 running sum
 * with kk ascending; P takes S's ir and jc unchanged.  Threading follows
 * MatFunctions.DDS (MatFunctions.scala:1634-1644): contiguous column ranges.
 * The value is stored (not accumulated), as DDShelper does. */
void oracle_dds(int k, int n, const float *A, const float *B, const int32_t *ir,
                const int32_t *jc, float *P, int nthreads) {
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for num_threads(nthreads) schedule(static, 1)
    for (int t = 0; t < nthreads; t++) {
        int istart = (int)((int64_t)t * n / nthreads);
        int iend = (int)((int64_t)(t + 1) * n / nthreads);
        for (int i = istart; i < iend; i++) {
            const float *b = B + (size_t)i * k;
            for (int j = jc[i]; j < jc[i + 1]; j++) {
                const float *a = A + (size_t)ir[j] * k;
                float dsum = 0.0f;
                for (int kk = 0; kk < k; kk++) {
                    float prod = a[kk] * b[kk];
                    dsum = dsum + prod;
                }
                P[j] = dsum;
            }
        }
    }
}

/* fp64 companions: same loops with double accumulation, used only to budget
 * rounding error (both the fp32 oracle and the GPU result are compared to
 * these).  They also return sum |term| per output element, the scale that the
 * relative tolerance is taken against. */
void oracle_dsmult_f64(int k, int n, const float *A, const float *data, const int32_t *ir,
                       const int32_t *jc, double *C, double *Cabs, int nthreads) {
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for num_threads(nthreads) schedule(dynamic, 64)
    for (int i = 0; i < n; i++) {
        double *out = C + (size_t)i * k;
        double *oab = Cabs + (size_t)i * k;
        for (int j = jc[i]; j < jc[i + 1]; j++) {
            double dval = data[j];
            const float *a = A + (size_t)ir[j] * k;
            for (int kk = 0; kk < k; kk++) {
                double p = (double)a[kk] * dval;
                out[kk] += p;
                oab[kk] += p < 0 ? -p : p;
            }
        }
    }
}

void oracle_dsmultT_f64(int k, int n, const float *B, const float *data, const int32_t *ir,
                        const int32_t *jc, double *C, double *Cabs, int nthreads) {
    int nt = nthreads < 1 ? 1 : nthreads;
    if (nt > k) nt = k;
#pragma omp parallel for num_threads(nt) schedule(static, 1)
    for (int t = 0; t < nt; t++) {
        int kstart = (int)((int64_t)k * t / nt);
        int kend = (int)((int64_t)k * (t + 1) / nt);
        for (int i = 0; i < n; i++) {
            const float *b = B + (size_t)i * k;
            for (int j = jc[i]; j < jc[i + 1]; j++) {
                double dval = data[j];
                double *out = C + (size_t)ir[j] * k;
                double *oab = Cabs + (size_t)ir[j] * k;
                for (int kk = kstart; kk < kend; kk++) {
                    double p = (double)b[kk] * dval;
                    out[kk] += p;
                    oab[kk] += p < 0 ? -p : p;
                }
            }
        }
    }
}

void oracle_dds_f64(int k, int n, const float *A, const float *B, const int32_t *ir,
                    const int32_t *jc, double *P, double *Pabs, int nthreads) {
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for num_threads(nthreads) schedule(dynamic, 64)
    for (int i = 0; i < n; i++) {
        const float *b = B + (size_t)i * k;
        for (int j = jc[i]; j < jc[i + 1]; j++) {
            const float *a = A + (size_t)ir[j] * k;
            double s = 0.0, sa = 0.0;
            for (int kk = 0; kk < k; kk++) {
                double p = (double)a[kk] * (double)b[kk];
                s += p;
                sa += p < 0 ? -p : p;
            }
            P[j] = s;
            Pabs[j] = sa;
        }
    }
}

/* SparseMat.uncompressInds, src/main/scala/BIDMat/SparseMat.scala:870-883
 * (0-based): ic[j] = i for j in [jc[i], jc[i+1]). */
void oracle_uncompress_inds(const int32_t *jc, int n, int32_t *ic) {
    for (int i = 0; i < n; i++)
        for (int j = jc[i]; j < jc[i + 1]; j++) ic[j] = i;
}

/* SparseMat.compressInds, src/main/scala/BIDMat/SparseMat.scala:857-868
 * (0-based): jc[i+1] = number of entries with ic <= i. */
void oracle_compress_inds(const int32_t *ic, int n, int32_t nnz, int32_t *jc) {
    jc[0] = 0;
    int32_t j = 0;
    for (int i = 0; i < n; i++) {
        while (j < nnz && ic[j] <= i) j++;
        jc[i + 1] = j;
    }
}

/* SparseMat.check, src/main/scala/BIDMat/SparseMat.scala:710-740 (0-based).
 * Returns 0 when the CSC invariants hold, else a small positive code naming the
 * first violated rule. */
int oracle_check_csc(int m, int n, int32_t nnz, const int32_t *ir, const int32_t *jc) {
    if (jc[0] != 0) return 1;
    for (int i = 0; i < n; i++) {
        if (jc[i] > jc[i + 1]) return 2;
        for (int j = jc[i]; j < jc[i + 1] - 1; j++) {
            if (ir[j + 1] <= ir[j]) return 3;
            if (ir[j] < 0) return 4;
            if (ir[j + 1] >= m) return 5;
        }
    }
    if (jc[n] != nnz) return 6;
    return 0;
}

/* Double-precision inputs and outputs: the same three loops on doubles, the CPU
 * counterpart of BIDMat's GDMat / GSDMat path.  A*S and B*^S are pinned
 * bit-exactly to the reference's own dmcscm / dmcsrm
 * (jni/src/BIDMat_SPBLAS.c:294-360); DDS on doubles is unpinned like its fp32 twin. */
void oracle_dsmult_d(int k, int n, const double *A, const double *data, const int32_t *ir,
                     const int32_t *jc, double *C, int nthreads) {
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for num_threads(nthreads) schedule(static, 1)
    for (int t = 0; t < nthreads; t++) {
        int istart = (int)((int64_t)t * n / nthreads);
        int iend = (int)((int64_t)(t + 1) * n / nthreads);
        for (int i = istart; i < iend; i++) {
            double *out = C + (size_t)i * k;
            for (int j = jc[i]; j < jc[i + 1]; j++) {
                double dval = data[j];
                const double *a = A + (size_t)ir[j] * k;
                for (int kk = 0; kk < k; kk++) {
                    double prod = a[kk] * dval;
                    out[kk] = out[kk] + prod;
                }
            }
        }
    }
}

void oracle_dsmultT_d(int k, int n, const double *B, const double *data, const int32_t *ir,
                      const int32_t *jc, double *C) {
    for (int i = 0; i < n; i++) {
        const double *b = B + (size_t)i * k;
        for (int j = jc[i]; j < jc[i + 1]; j++) {
            double dval = data[j];
            double *out = C + (size_t)ir[j] * k;
            for (int kk = 0; kk < k; kk++) {
                double prod = b[kk] * dval;
                out[kk] = out[kk] + prod;
            }
        }
    }
}

void oracle_dds_d(int k, int n, const double *A, const double *B, const int32_t *ir,
                  const int32_t *jc, double *P) {
    for (int i = 0; i < n; i++) {
        const double *b = B + (size_t)i * k;
        for (int j = jc[i]; j < jc[i + 1]; j++) {
            const double *a = A + (size_t)ir[j] * k;
            double dsum = 0.0;
            for (int kk = 0; kk < k; kk++) {
                double prod = a[kk] * b[kk];
                dsum = dsum + prod;
            }
            P[j] = dsum;
        }
    }
}
