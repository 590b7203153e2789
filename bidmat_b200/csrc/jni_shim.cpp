// JNI entry points that rebind BIDMat's native methods for the sparse-dense
// path onto this library.  Compiled only when a JDK's <jni.h> is available
// (the build passes -DBIDMAT_B200_WITH_JNI=1 then); the C ABI underneath is
// what the test-suite exercises.
//
// Each function decodes jcuda.Pointer arguments exactly as BIDMat's glue does
// (address = NativePointerObject.nativePointer + Pointer.byteOffset,
// jni/src/PointerUtils.cpp:353-363) and forwards to the C ABI.  Two ways to
// use it:
//   (i)  link this object into libbidmatcuda in place of the four launchers of
//        jni/src/Arith.cu: the exported Java_edu_berkeley_bid_CUMAT_* symbols
//        below then replace those of jni/src/BIDMat_CUMAT.cpp:722-798;
//   (ii) load this library next to the stock one and let JNI_OnLoad re-register
//        the four natives of edu.berkeley.bid.CUMAT (RegisterNatives overrides
//        the bindings made by name lookup).
#if defined(BIDMAT_B200_WITH_JNI)
#include <jni.h>

#include "../../include/bidmat_b200.h"

namespace {

jfieldID g_native_pointer = nullptr;  // jcuda.NativePointerObject.nativePointer (J)
jfieldID g_byte_offset = nullptr;     // jcuda.Pointer.byteOffset (J)

bool init_field_ids(JNIEnv *env) {
    if (g_native_pointer && g_byte_offset) return true;
    jclass npo = env->FindClass("jcuda/NativePointerObject");
    if (!npo) return false;
    g_native_pointer = env->GetFieldID(npo, "nativePointer", "J");
    jclass ptr = env->FindClass("jcuda/Pointer");
    if (!ptr) return false;
    g_byte_offset = env->GetFieldID(ptr, "byteOffset", "J");
    return g_native_pointer && g_byte_offset;
}

void *device_address(JNIEnv *env, jobject p) {
    if (!p) return nullptr;
    const jlong base = env->GetLongField(p, g_native_pointer);
    const jlong off = env->GetLongField(p, g_byte_offset);
    return reinterpret_cast<void *>(base + off);
}

}  // namespace

extern "C" {

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_dsmult(JNIEnv *env, jclass, jint nrows, jint ncols, jint nnz,
                                                         jobject jA, jobject jBdata, jobject jBir, jobject jBic,
                                                         jobject jC) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_dsmult(nrows, ncols, nnz, (const float *)device_address(env, jA),
                              (const float *)device_address(env, jBdata), (const int *)device_address(env, jBir),
                              (const int *)device_address(env, jBic), (float *)device_address(env, jC));
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_dsmultT(JNIEnv *env, jclass, jint nrows, jint ncols, jint nnz,
                                                          jobject jA, jobject jBdata, jobject jBir, jobject jBic,
                                                          jobject jC) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_dsmultT(nrows, ncols, nnz, (const float *)device_address(env, jA),
                               (const float *)device_address(env, jBdata), (const int *)device_address(env, jBir),
                               (const int *)device_address(env, jBic), (float *)device_address(env, jC));
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_dds(JNIEnv *env, jclass, jint nrows, jint nnz, jobject jA,
                                                      jobject jB, jobject jCir, jobject jCic, jobject jP) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_dds(nrows, nnz, (const float *)device_address(env, jA), (const float *)device_address(env, jB),
                           (const int *)device_address(env, jCir), (const int *)device_address(env, jCic),
                           (float *)device_address(env, jP));
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_dds0(JNIEnv *env, jclass, jint nrows, jint ncols, jobject jA,
                                                       jobject jB, jobject jCir, jobject jCjc, jobject jP) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_dds0(nrows, ncols, (const float *)device_address(env, jA),
                            (const float *)device_address(env, jB), (const int *)device_address(env, jCir),
                            (const int *)device_address(env, jCjc), (float *)device_address(env, jP));
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_dsmulttune(JNIEnv *env, jclass c, jint nrows, jint ncols, jint nnz,
                                                             jobject jA, jobject jBdata, jobject jBir, jobject jBic,
                                                             jobject jC, jint, jint) {
    return Java_edu_berkeley_bid_CUMAT_dsmult(env, c, nrows, ncols, nnz, jA, jBdata, jBir, jBic, jC);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_dsmultxtune(JNIEnv *env, jclass c, jint nrows, jint ncols,
                                                              jint nnz, jobject jA, jobject jBdata, jobject jBir,
                                                              jobject jBic, jobject jC, jint, jint, jint) {
    return Java_edu_berkeley_bid_CUMAT_dsmult(env, c, nrows, ncols, nnz, jA, jBdata, jBir, jBic, jC);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_dsmultTile(JNIEnv *env, jclass, jint nr, jint nc, jint kk, jint nnz,
                                                             jobject jA, jint lda, jobject jBdata, jobject jBir,
                                                             jobject jBic, jint broff, jint bcoff, jobject jC, jint ldc,
                                                             jint transpose) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_dsmultTile(nr, nc, kk, nnz, (const float *)device_address(env, jA), lda,
                                  (const float *)device_address(env, jBdata), (const int *)device_address(env, jBir),
                                  (const int *)device_address(env, jBic), broff, bcoff,
                                  (float *)device_address(env, jC), ldc, transpose);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_spsum(JNIEnv *env, jclass, jint nrows, jint ncols, jint nnz,
                                                        jobject jAir, jobject jAic, jobject jP, jobject jB, jint n) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_spsum(nrows, ncols, nnz, (const int *)device_address(env, jAir),
                             (const int *)device_address(env, jAic), (const float *)device_address(env, jP),
                             (float *)device_address(env, jB), n);
}

// Edge operators: sdoprow / sdopcol are the fp32 natives; the double-precision ones are
// separate natives, sdopdrow / sdopdcol (CUMAT.java:137,141), bound below.
JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_sdoprow(JNIEnv *env, jclass, jint nrows, jint ncols, jint nnz,
                                                          jobject jA, jobject jAic, jobject jB, jint len, jint opn) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_sdoprow(nrows, ncols, nnz, (float *)device_address(env, jA),
                               (const int *)device_address(env, jAic), (const float *)device_address(env, jB), len, opn);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_sdopcol(JNIEnv *env, jclass, jint nrows, jint ncols, jint nnz,
                                                          jobject jA, jobject jAir, jobject jB, jint len, jint opn) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_sdopcol(nrows, ncols, nnz, (float *)device_address(env, jA),
                               (const int *)device_address(env, jAir), (const float *)device_address(env, jB), len, opn);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_sdopdrow(JNIEnv *env, jclass, jint nrows, jint ncols, jint nnz,
                                                           jobject jA, jobject jAic, jobject jB, jint len, jint opn) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_sdoprow_f64(nrows, ncols, nnz, (double *)device_address(env, jA),
                                   (const int *)device_address(env, jAic), (const double *)device_address(env, jB),
                                   len, opn);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMAT_sdopdcol(JNIEnv *env, jclass, jint nrows, jint ncols, jint nnz,
                                                           jobject jA, jobject jAir, jobject jB, jint len, jint opn) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_sdopcol_f64(nrows, ncols, nnz, (double *)device_address(env, jA),
                                   (const int *)device_address(env, jAir), (const double *)device_address(env, jB),
                                   len, opn);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMATD_spsum(JNIEnv *env, jclass, jint nrows, jint ncols, jint nnz,
                                                         jobject jAir, jobject jAic, jobject jP, jobject jB, jint n) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_spsum_f64(nrows, ncols, nnz, (const int *)device_address(env, jAir),
                                 (const int *)device_address(env, jAic), (const double *)device_address(env, jP),
                                 (double *)device_address(env, jB), n);
}

// Double-precision natives of edu.berkeley.bid.CUMATD (CUMATD.java:51,57,71,89,91).
JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMATD_dsmult(JNIEnv *env, jclass, jint nrows, jint ncols, jint nnz,
                                                          jobject jA, jobject jBdata, jobject jBir, jobject jBic,
                                                          jobject jC) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_dsmult_f64(nrows, ncols, nnz, (const double *)device_address(env, jA),
                                  (const double *)device_address(env, jBdata), (const int *)device_address(env, jBir),
                                  (const int *)device_address(env, jBic), (double *)device_address(env, jC));
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMATD_dsmultT(JNIEnv *env, jclass, jint nrows, jint ncols, jint nnz,
                                                           jobject jA, jobject jBdata, jobject jBir, jobject jBic,
                                                           jobject jC) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_dsmultT_f64(nrows, ncols, nnz, (const double *)device_address(env, jA),
                                   (const double *)device_address(env, jBdata), (const int *)device_address(env, jBir),
                                   (const int *)device_address(env, jBic), (double *)device_address(env, jC));
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMATD_dds(JNIEnv *env, jclass, jint nrows, jint nnz, jobject jA,
                                                       jobject jB, jobject jCir, jobject jCic, jobject jP) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_dds_f64(nrows, nnz, (const double *)device_address(env, jA),
                               (const double *)device_address(env, jB), (const int *)device_address(env, jCir),
                               (const int *)device_address(env, jCic), (double *)device_address(env, jP));
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_CUMATD_dds0(JNIEnv *env, jclass, jint nrows, jint ncols, jobject jA,
                                                        jobject jB, jobject jCir, jobject jCjc, jobject jP) {
    if (!init_field_ids(env)) return 1;
    return bidmat_b200_dds0_f64(nrows, ncols, (const double *)device_address(env, jA),
                                (const double *)device_address(env, jB), (const int *)device_address(env, jCir),
                                (const int *)device_address(env, jCjc), (double *)device_address(env, jP));
}

// Route (ii): rebind the four natives when this library is loaded by System.load.
JNIEXPORT jint JNICALL JNI_OnLoad(JavaVM *vm, void *) {
    JNIEnv *env = nullptr;
    if (vm->GetEnv(reinterpret_cast<void **>(&env), JNI_VERSION_1_6) != JNI_OK) return JNI_ERR;
    if (!init_field_ids(env)) return JNI_ERR;
    jclass cumat = env->FindClass("edu/berkeley/bid/CUMAT");
    if (!cumat) {            // class not loaded yet: name lookup will bind the exports above
        env->ExceptionClear();
        return JNI_VERSION_1_6;
    }
    static const char *P = "Ljcuda/Pointer;";
    (void)P;
    JNINativeMethod m[] = {
        {(char *)"dsmult", (char *)"(IIILjcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;)I",
         (void *)Java_edu_berkeley_bid_CUMAT_dsmult},
        {(char *)"dsmultT", (char *)"(IIILjcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;)I",
         (void *)Java_edu_berkeley_bid_CUMAT_dsmultT},
        {(char *)"dds", (char *)"(IILjcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;)I",
         (void *)Java_edu_berkeley_bid_CUMAT_dds},
        {(char *)"dds0", (char *)"(IILjcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;Ljcuda/Pointer;)I",
         (void *)Java_edu_berkeley_bid_CUMAT_dds0},
    };
    if (env->RegisterNatives(cumat, m, 4) != 0) return JNI_ERR;
    return JNI_VERSION_1_6;
}

}  // extern "C"
#endif  // BIDMAT_B200_WITH_JNI
