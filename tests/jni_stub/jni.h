/*
 * TEST INFRASTRUCTURE.  A stand-in for the JDK's <jni.h> with just the C++
 * declarations that bidmat_b200/csrc/jni_shim.cpp and nccl_jni_shim.cpp use, so that the shims can be
 * compile-checked where no JDK is installed (tests/test_jni_shim.py).  It is
 * never used to build the product library.
 */
#ifndef TESTS_JNI_STUB_JNI_H
#define TESTS_JNI_STUB_JNI_H
#include <cstdint>

typedef int32_t jint;
typedef int64_t jlong;
class _jobject {};
typedef _jobject *jobject;
typedef jobject jclass;
typedef jobject jobjectArray;
typedef jint jsize;
struct _jfieldID;
typedef _jfieldID *jfieldID;

#define JNIEXPORT __attribute__((visibility("default")))
#define JNICALL
#define JNI_OK 0
#define JNI_ERR (-1)
#define JNI_VERSION_1_6 0x00010006

struct JNINativeMethod {
    char *name;
    char *signature;
    void *fnPtr;
};

struct JNIEnv {
    jclass FindClass(const char *name);
    jfieldID GetFieldID(jclass clazz, const char *name, const char *sig);
    jlong GetLongField(jobject obj, jfieldID field);
    void SetLongField(jobject obj, jfieldID field, jlong value);
    jsize GetArrayLength(jobjectArray array);
    jobject GetObjectArrayElement(jobjectArray array, jsize index);
    void ExceptionClear();
    jint RegisterNatives(jclass clazz, const JNINativeMethod *methods, jint count);
};

struct JavaVM {
    jint GetEnv(void **penv, jint version);
};
#endif
