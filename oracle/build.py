"""Build recipe for the CPU checker (test infrastructure, not product code).

Produces, beside this file:
  liboracle.so             the C restatement in spdense_oracle.c (strict fp32, plain x86-64)
  liboracle_native_*.so    the same file built -O3 -march=native for the host it is
                           built on (the name carries a hash of the CPU's feature
                           flags, so a copy made on another machine is not picked up);
                           same bits (tests/test_oracle.py), used for the timed CPU baseline
  _ref/libspblas_ref.so    the reference's own jni/src/BIDMat_SPBLAS.c, compiled
                           from the reference checkout where it lies together with
                           ref_driver.c, against the stand-in headers in refshim/
  _ref/libarith_ref.so     the reference's own CUDA launchers and kernels
                           (jni/src/Arith.cu), compiled for sm_100a from the
                           checkout where it lies together with ref_gpu_driver.cu,
                           with refshim/legacy_shuffle.h force-included
The two _ref libraries are only built when a reference checkout is present; no
reference file is ever copied into this repository.

The reference checkout is taken from the argument, else from the environment
variable BIDMAT_REFERENCE_ROOT, else from a directory named `reference` beside
the repository.

Run as ``python oracle/build.py [reference_root]``.
"""
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libspblas_ref.so")
REF_GPU_SO = os.path.join(REF_DIR, "libarith_ref.so")


def reference_root(explicit=None):
    if explicit:
        return explicit
    env = os.environ.get("BIDMAT_REFERENCE_ROOT")
    if env:
        return env
    return os.path.normpath(os.path.join(HERE, "..", "..", "reference"))


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "spdense_oracle.c")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
           "-fno-fast-math", "-o", ORACLE_SO, src]
    subprocess.check_call(cmd)
    return ORACLE_SO


def _cpu_flags_tag():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                return hashlib.sha1(line.encode()).hexdigest()[:10]
    except OSError:
        pass
    return "generic"


def build_oracle_native(force=False):
    """-O3 -march=native build of the same source for the machine this runs on.
    Contraction stays off, so every product is rounded before it is added and the
    bits do not depend on the vector width.  Returns None when it cannot be built."""
    src = os.path.join(HERE, "spdense_oracle.c")
    out = os.path.join(HERE, "liboracle_native_%s.so" % _cpu_flags_tag())
    if not force and _newer(out, [src]):
        return out
    cmd = ["gcc", "-O3", "-march=native", "-std=c11", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
           "-fno-fast-math", "-o", out, src]
    try:
        subprocess.check_call(cmd, stderr=subprocess.DEVNULL)
    except (OSError, subprocess.CalledProcessError):
        return None
    return out


def build_reference(root=None, force=False):
    """Compile the reference's C loops; returns the .so path or None when no
    reference checkout is available (the prebuilt file, if any, is kept)."""
    root = reference_root(root)
    ref_src = os.path.join(root, "jni", "src", "BIDMat_SPBLAS.c")
    if not os.path.exists(ref_src):
        return REF_SO if os.path.exists(REF_SO) else None
    drv = os.path.join(HERE, "ref_driver.c")
    shim = os.path.join(HERE, "refshim")
    os.makedirs(REF_DIR, exist_ok=True)
    if not force and _newer(REF_SO, [ref_src, drv, os.path.join(shim, "jni.h")]):
        return REF_SO
    # -O2 without -march: no FMA instructions exist in the baseline x86-64 ISA,
    # so the reference's "Cp[k] += bv * Ap[k]" rounds twice, as on the JVM.
    cmd = ["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-w",
           "-I", shim, "-o", REF_SO, drv, ref_src]
    subprocess.check_call(cmd)
    return REF_SO


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def build_reference_gpu(root=None, force=False):
    """Compile the reference's CUDA launchers (dsmult, dsmultT, dds, dds0, spsum and the
    rest of jni/src/Arith.cu) for sm_100a; returns the .so path or None when there is no
    reference checkout or no nvcc (a prebuilt file, if any, is kept)."""
    root = reference_root(root)
    ref_src = os.path.join(root, "jni", "src", "Arith.cu")
    inc = os.path.join(root, "jni", "include")
    nvcc = _nvcc()
    if not os.path.exists(ref_src) or nvcc is None:
        return REF_GPU_SO if os.path.exists(REF_GPU_SO) else None
    drv = os.path.join(HERE, "ref_gpu_driver.cu")
    shim = os.path.join(HERE, "refshim", "legacy_shuffle.h")
    os.makedirs(REF_DIR, exist_ok=True)
    if not force and _newer(REF_GPU_SO, [ref_src, drv, shim]):
        return REF_GPU_SO
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-w", "-I", inc, "-include", shim,
           "-shared", "-Xcompiler", "-fPIC", "-o", REF_GPU_SO, drv, ref_src]
    subprocess.check_call(cmd)
    return REF_GPU_SO


def build_all(root=None, force=False):
    return build_oracle(force), build_reference(root, force), build_reference_gpu(root, force)


if __name__ == "__main__":
    print(build_all(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
