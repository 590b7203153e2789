"""In-tree build of the CUDA library for sm_100a (nvcc cross-compiles without a GPU).

``python -m bidmat_b200.build`` writes bidmat_b200/lib/libbidmatcuda_b200.so.
The JNI shim (csrc/jni_shim.cpp) is compiled in only when a JDK's jni.h can be
found (JAVA_HOME or the usual /usr/lib/jvm locations).
"""
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
LIBNAME = "libbidmatcuda_b200.so"
LIBPATH = os.path.join(LIBDIR, LIBNAME)
COMPAT_OBJ = os.path.join(LIBDIR, "matkernel_compat.o")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def find_nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the library cannot be built")


def find_jni_include():
    roots = []
    if os.environ.get("JAVA_HOME"):
        roots.append(os.environ["JAVA_HOME"])
    roots += sorted(glob.glob("/usr/lib/jvm/*"))
    for r in roots:
        inc = os.path.join(r, "include")
        if os.path.exists(os.path.join(inc, "jni.h")):
            return [inc, os.path.join(inc, "linux")]
    return None


def find_nccl():
    """(include dir, library dir) of an NCCL 2 installation, or None."""
    for inc, lib in (("/usr/include", "/usr/lib/x86_64-linux-gnu"), ("/usr/local/cuda/include", "/usr/local/cuda/lib64")):
        if os.path.exists(os.path.join(inc, "nccl.h")) and glob.glob(os.path.join(lib, "libnccl.so*")):
            return inc, lib
    return None


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale():
    if not os.path.exists(LIBPATH):
        return True
    t = os.path.getmtime(LIBPATH)
    deps = glob.glob(os.path.join(CSRC, "*")) + [os.path.join(PKG, "..", "include", "bidmat_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not _stale():
        return LIBPATH
    os.makedirs(LIBDIR, exist_ok=True)
    cmd = [find_nvcc()] + ARCH_FLAGS + [
        "-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
        "-I", os.path.join(PKG, "..", "include"), "-o", LIBPATH]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    srcs = sources()
    jni = find_jni_include()
    if jni:
        for d in jni:
            cmd += ["-I", d]
        cmd += ["-DBIDMAT_B200_WITH_JNI=1"]
        srcs.append(os.path.join(CSRC, "jni_shim.cpp"))
        nccl = find_nccl()
        if nccl:      # the edu.berkeley.bid.NCCL natives on NCCL 2
            cmd += ["-I", nccl[0], "-L", nccl[1], "-lnccl", "-DBIDMAT_B200_WITH_NCCL=1"]
            srcs.append(os.path.join(CSRC, "nccl_jni_shim.cpp"))
    cmd += srcs
    subprocess.check_call(cmd)
    # MatKernel.hpp launcher names on top of the C ABI, for linking into BIDMat's own
    # libbidmatcuda (kept out of this library: see the file's header)
    cxx = shutil.which("g++")
    if cxx:
        subprocess.check_call([cxx, "-std=c++17", "-O2", "-c", "-fPIC", "-I", os.path.join(PKG, "..", "include"),
                               os.path.join(CSRC, "matkernel_compat.cpp"), "-o", COMPAT_OBJ])
    return LIBPATH


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
