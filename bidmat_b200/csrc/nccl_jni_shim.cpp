// JNI entry points of BIDMat's edu.berkeley.bid.NCCL class on top of NCCL 2.
//
// BIDMat's binding (jni/src/BIDMat_NCCL.cpp:57-90, src/main/java/edu/berkeley/bid/NCCL.java:22-33)
// was written for NCCL 1 and is driven by GFunctions.ncclAllReduce
// (src/main/scala/BIDMat/GFunctions.scala:175-203): ONE host thread creates a
// communicator per GPU with ncclCommInitAll, calls ncclAllReduce once per GPU with the
// datatype literal 3 ("float" in NCCL 1's enumeration), synchronises the streams and
// destroys the communicators again, on every call.  Against NCCL 2 that sequence needs
// three things, which this shim supplies:
//   * datatype numbers are translated from NCCL 1's enumeration (char, int, half,
//     float, double, int64, uint64) to NCCL 2's; 3 becomes ncclFloat32;
//   * the per-GPU calls of one host thread are wrapped in ncclGroupStart / ncclGroupEnd:
//     the group opens at the first call on a set of communicators and closes when every
//     communicator of the set has been used once (without it the first call would wait
//     for the others and never return);
//   * communicators are kept alive: ncclCommInitAll for a device count seen before hands
//     out the communicators made the first time and ncclCommDestroy only detaches the Java
//     object, so the cost of communicator set-up is paid once per process, not per call.
// Callers that drive one GPU per host thread must not use this path (NCCL groups are per
// thread); they can sum with bidmat_b200_peer_allreduce_sum instead.
//
// Compiled only when a JDK's <jni.h> and NCCL's <nccl.h> are available
// (-DBIDMAT_B200_WITH_JNI=1 -DBIDMAT_B200_WITH_NCCL=1).
#if defined(BIDMAT_B200_WITH_JNI) && defined(BIDMAT_B200_WITH_NCCL)
#include <jni.h>
#include <nccl.h>

#include <map>
#include <mutex>
#include <vector>

namespace {

struct Clique {
    std::vector<ncclComm_t> comms;
    int pending = 0;          // calls made inside the open group
};

std::mutex g_mu;
std::map<int, Clique> g_cliques;             // by number of devices
std::map<ncclComm_t, Clique *> g_owner;

// NCCL 1 enumeration (the reference passes these numbers) -> NCCL 2
bool translate_type(int nccl1, ncclDataType_t *out) {
    switch (nccl1) {
        case 0: *out = ncclInt8; return true;      // ncclChar
        case 1: *out = ncclInt32; return true;     // ncclInt
        case 2: *out = ncclFloat16; return true;   // ncclHalf
        case 3: *out = ncclFloat32; return true;   // ncclFloat: what GFunctions.ncclAllReduce passes
        case 4: *out = ncclFloat64; return true;   // ncclDouble
        case 5: *out = ncclInt64; return true;
        case 6: *out = ncclUint64; return true;
        default: return false;
    }
}

jfieldID handle_field(JNIEnv *env, jclass clazz) { return env->GetFieldID(clazz, "handle", "J"); }

void *pointer_of(JNIEnv *env, jobject p) {         // jcuda.Pointer: nativePointer + byteOffset
    if (!p) return nullptr;
    jclass npo = env->FindClass("jcuda/NativePointerObject");
    jclass ptr = env->FindClass("jcuda/Pointer");
    if (!npo || !ptr) return nullptr;
    const jlong base = env->GetLongField(p, env->GetFieldID(npo, "nativePointer", "J"));
    const jlong off = env->GetLongField(p, env->GetFieldID(ptr, "byteOffset", "J"));
    return reinterpret_cast<void *>(base + off);
}

void *native_pointer_of(JNIEnv *env, jobject p) {  // jcuda.runtime.cudaStream_t: nativePointer only
    if (!p) return nullptr;
    jclass npo = env->FindClass("jcuda/NativePointerObject");
    if (!npo) return nullptr;
    return reinterpret_cast<void *>(env->GetLongField(p, env->GetFieldID(npo, "nativePointer", "J")));
}

}  // namespace

extern "C" {

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_NCCL_hasNCCL(JNIEnv *, jclass) { return 1; }

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_NCCL_ncclCommInitAll(JNIEnv *env, jclass clazz, jobjectArray jcomms) {
    const jsize len = env->GetArrayLength(jcomms);
    if (len <= 0) return (jint)ncclInvalidArgument;
    std::lock_guard<std::mutex> g(g_mu);
    Clique &cl = g_cliques[(int)len];
    if (cl.comms.empty()) {
        cl.comms.resize((size_t)len);
        const ncclResult_t st = ncclCommInitAll(cl.comms.data(), (int)len, nullptr);
        if (st != ncclSuccess) { cl.comms.clear(); return (jint)st; }
        for (ncclComm_t c : cl.comms) g_owner[c] = &cl;
    }
    const jfieldID fid = handle_field(env, clazz);
    for (jsize i = 0; i < len; i++)
        env->SetLongField(env->GetObjectArrayElement(jcomms, i), fid, (jlong) reinterpret_cast<intptr_t>(cl.comms[(size_t)i]));
    return (jint)ncclSuccess;
}

JNIEXPORT void JNICALL Java_edu_berkeley_bid_NCCL_ncclCommDestroy(JNIEnv *env, jclass clazz, jobject jcomm) {
    // the communicator stays in the cache for the next ncclCommInitAll; only the Java object lets go of it
    env->SetLongField(jcomm, handle_field(env, clazz), (jlong)0);
}

JNIEXPORT jint JNICALL Java_edu_berkeley_bid_NCCL_ncclAllReduce(JNIEnv *env, jclass clazz, jobject jsend, jobject jrecv,
                                                               jint count, jint datatype, jint op, jobject jcomm,
                                                               jobject jstream) {
    ncclDataType_t type;
    if (!translate_type((int)datatype, &type) || op < 0 || op > 3 || count < 0) return (jint)ncclInvalidArgument;
    ncclComm_t comm = reinterpret_cast<ncclComm_t>((intptr_t)env->GetLongField(jcomm, handle_field(env, clazz)));
    if (!comm) return (jint)ncclInvalidArgument;
    void *send = pointer_of(env, jsend);
    void *recv = pointer_of(env, jrecv);
    cudaStream_t stream = static_cast<cudaStream_t>(native_pointer_of(env, jstream));
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_owner.find(comm);
    if (it == g_owner.end()) return (jint)ncclInvalidArgument;
    Clique *cl = it->second;
    ncclResult_t st = ncclSuccess;
    if (cl->pending == 0) st = ncclGroupStart();
    if (st == ncclSuccess)
        st = ncclAllReduce(send, recv, (size_t)count, type, (ncclRedOp_t)op, comm, stream);
    cl->pending++;
    if (cl->pending == (int)cl->comms.size() || st != ncclSuccess) {
        const ncclResult_t end = ncclGroupEnd();
        cl->pending = 0;
        if (st == ncclSuccess) st = end;
    }
    return (jint)st;
}

}  // extern "C"
#endif  // BIDMAT_B200_WITH_JNI && BIDMAT_B200_WITH_NCCL
