/*
 * TEST INFRASTRUCTURE.  Plain-pointer entry points over the reference's own C
 * loops for A*S and B*^S.  oracle/build.py compiles this file together with
 * jni/src/BIDMat_SPBLAS.c taken from the reference tree where it lies (never
 * copied), against the stand-in headers in refshim/.  The JNI environment
 * handed to the reference functions is a table of pass-through accessors: a
 * Java array handle is the buffer's own address.
 *
 *   ref_smcscm -> Java_edu_berkeley_bid_SPBLAS_smcscm (BIDMat_SPBLAS.c:364-395)
 *   ref_smcsrm -> Java_edu_berkeley_bid_SPBLAS_smcsrm (BIDMat_SPBLAS.c:397-427)
 */
#include <jni.h>
#include <stddef.h>

JNIEXPORT void JNICALL Java_edu_berkeley_bid_SPBLAS_smcscm(JNIEnv *, jobject, jint, jint, jfloatArray,
                                                          jint, jfloatArray, jintArray, jintArray,
                                                          jfloatArray, jint);
JNIEXPORT void JNICALL Java_edu_berkeley_bid_SPBLAS_smcsrm(JNIEnv *, jobject, jint, jint, jfloatArray,
                                                          jint, jfloatArray, jintArray, jintArray,
                                                          jfloatArray, jint);

static void *pass_get(JNIEnv *env, jarray array, jboolean *is_copy) {
    (void)env;
    (void)is_copy; /* the reference passes JNI_FALSE (0) here, i.e. a null pointer */
    return array;
}
static void pass_release(JNIEnv *env, jarray array, void *carray, jint mode) {
    (void)env; (void)array; (void)carray; (void)mode;
}
static const char *pass_chars(JNIEnv *env, jstring s, jboolean *is_copy) {
    (void)env; (void)is_copy;
    return (const char *)s;
}
static void pass_release_chars(JNIEnv *env, jstring s, const char *c) {
    (void)env; (void)s; (void)c;
}

static const struct JNINativeInterface_ table = {pass_get, pass_release, pass_chars, pass_release_chars};

/* C(k x n) += A(k x m) * S, S = (data, ir, jc) CSC; index base taken from jc[0]
 * exactly as the reference does. */
void ref_smcscm(int k, int n, float *A, float *data, int *ir, int *jc, float *C) {
    JNIEnv env = &table;
    Java_edu_berkeley_bid_SPBLAS_smcscm(&env, NULL, k, n, A, k, data, ir, jc, C, k);
}

/* C(k x m) += B(k x n) * S^T. */
void ref_smcsrm(int k, int n, float *B, float *data, int *ir, int *jc, float *C) {
    JNIEnv env = &table;
    Java_edu_berkeley_bid_SPBLAS_smcsrm(&env, NULL, k, n, B, k, data, ir, jc, C, k);
}

JNIEXPORT void JNICALL Java_edu_berkeley_bid_SPBLAS_dmcscm(JNIEnv *, jobject, jint, jint, jdoubleArray,
                                                          jint, jdoubleArray, jintArray, jintArray,
                                                          jdoubleArray, jint);
JNIEXPORT void JNICALL Java_edu_berkeley_bid_SPBLAS_dmcsrm(JNIEnv *, jobject, jint, jint, jdoubleArray,
                                                          jint, jdoubleArray, jintArray, jintArray,
                                                          jdoubleArray, jint);

/* Double-precision twins: dmcscm / dmcsrm (BIDMat_SPBLAS.c:294-360). */
void ref_dmcscm(int k, int n, double *A, double *data, int *ir, int *jc, double *C) {
    JNIEnv env = &table;
    Java_edu_berkeley_bid_SPBLAS_dmcscm(&env, NULL, k, n, A, k, data, ir, jc, C, k);
}

void ref_dmcsrm(int k, int n, double *B, double *data, int *ir, int *jc, double *C) {
    JNIEnv env = &table;
    Java_edu_berkeley_bid_SPBLAS_dmcsrm(&env, NULL, k, n, B, k, data, ir, jc, C, k);
}
