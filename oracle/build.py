"""Build recipe for the CPU checker (test infrastructure, not product code).

Produces, beside this file:
  liboracle.so          the C restatement in spdense_oracle.c (strict fp32)
  _ref/libspblas_ref.so the reference's own jni/src/BIDMat_SPBLAS.c, compiled
                        from the reference checkout where it lies together with
                        ref_driver.c, against the stand-in headers in refshim/.
                        Only built when a reference checkout is present; the
                        file is never copied into this repository.

Run as ``python oracle/build.py [reference_root]``.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libspblas_ref.so")
DEFAULT_REFERENCE_ROOT = os.environ.get("BIDMAT_REFERENCE_ROOT", "/root/reference")


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


def build_reference(reference_root=DEFAULT_REFERENCE_ROOT, force=False):
    """Compile the reference's C loops; returns the .so path or None when no
    reference checkout is available (the prebuilt file, if any, is kept)."""
    ref_src = os.path.join(reference_root, "jni", "src", "BIDMat_SPBLAS.c")
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


def build_all(reference_root=DEFAULT_REFERENCE_ROOT, force=False):
    return build_oracle(force), build_reference(reference_root, force)


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE_ROOT
    print(build_all(root, force=True))
