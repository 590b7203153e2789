/*
 * TEST INFRASTRUCTURE.  Minimal stand-in for the JDK's <jni.h>, written for
 * this repository because no JDK is installed where the oracle is built.  It
 * declares only what BIDMat's jni/src/BIDMat_SPBLAS.c touches when compiled
 * with gcc (the non-MKL half of that file): the scalar and handle typedefs and
 * a function table holding the four array/string accessors.  The driver in
 * ref_driver.c fills that table with pass-through functions, so an "array
 * handle" is simply the address of the caller's buffer.
 */
#ifndef ORACLE_REFSHIM_JNI_H
#define ORACLE_REFSHIM_JNI_H
#include <stdint.h>

typedef int32_t jint;
typedef int64_t jlong;
typedef float jfloat;
typedef double jdouble;
typedef unsigned char jboolean;
typedef void *jobject;
typedef jobject jarray;
typedef jobject jstring;
typedef jarray jintArray;
typedef jarray jfloatArray;
typedef jarray jdoubleArray;

#define JNI_FALSE 0
#define JNI_TRUE 1
#define JNIEXPORT __attribute__((visibility("default")))
#define JNICALL

struct JNINativeInterface_;
typedef const struct JNINativeInterface_ *JNIEnv;

struct JNINativeInterface_ {
    void *(*GetPrimitiveArrayCritical)(JNIEnv *env, jarray array, jboolean *isCopy);
    void (*ReleasePrimitiveArrayCritical)(JNIEnv *env, jarray array, void *carray, jint mode);
    const char *(*GetStringUTFChars)(JNIEnv *env, jstring str, jboolean *isCopy);
    void (*ReleaseStringUTFChars)(JNIEnv *env, jstring str, const char *chars);
};
#endif
