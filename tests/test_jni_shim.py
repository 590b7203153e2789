"""The JNI shim cannot be built where no JDK exists, so it is at least
compile-checked against a stand-in <jni.h> (tests/jni_stub) and its exported
symbol names are compared with the natives BIDMat declares
(src/main/java/edu/berkeley/bid/CUMAT.java:135-152, 209-213; CUMATD.java:51-91)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_jni_shim_compiles_and_exports_the_native_names(tmp_path):
    obj = str(tmp_path / "jni_shim.o")
    cmd = ["g++", "-std=c++17", "-c", "-fPIC", "-fvisibility=hidden", "-DBIDMAT_B200_WITH_JNI=1", "-Wall", "-Werror",
           "-I", os.path.join(ROOT, "tests", "jni_stub"), "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "bidmat_b200", "csrc", "jni_shim.cpp"), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    syms = subprocess.run(["nm", "-g", "--defined-only", obj], capture_output=True, text=True).stdout
    for name in ("CUMAT_dsmult", "CUMAT_dsmultT", "CUMAT_dds", "CUMAT_dds0", "CUMAT_dsmulttune", "CUMAT_dsmultxtune",
                 "CUMAT_dsmultTile", "CUMAT_spsum", "CUMAT_sdoprow", "CUMAT_sdopcol",
                 "CUMAT_sdopdrow", "CUMAT_sdopdcol", "CUMATD_spsum",
                 "CUMATD_dsmult", "CUMATD_dsmultT", "CUMATD_dds", "CUMATD_dds0"):
        assert ("Java_edu_berkeley_bid_" + name + "\n") in syms, name
    assert "JNI_OnLoad" in syms
    # everything the shim calls is declared in the public header
    undefined = subprocess.run(["nm", "-u", obj], capture_output=True, text=True).stdout
    from bidmat_b200 import _lib
    declared = set(_lib.declared_symbols())
    for line in undefined.splitlines():
        sym = line.split()[-1]
        if sym.startswith("bidmat_b200_"):
            assert sym in declared, sym


def _first_existing(paths):
    for p in paths:
        if os.path.exists(p):
            return p
    return None


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_nccl_jni_shim_compiles_against_nccl2(tmp_path):
    """The binding of edu.berkeley.bid.NCCL (NCCL.java:22-33, BIDMat_NCCL.cpp:57-90) on NCCL 2:
    compile-checked against the stand-in jni.h and the system's nccl.h; exports the four
    natives and calls the group API."""
    import glob
    nccl = _first_existing(["/usr/include/nccl.h"] + glob.glob(os.path.join(
        os.path.dirname(os.__file__), "site-packages", "nvidia", "nccl", "include", "nccl.h")))
    cuda = _first_existing(["/usr/local/cuda/include/cuda_runtime.h"])
    if nccl is None or cuda is None:
        pytest.skip("no nccl.h / cuda_runtime.h on this machine")
    obj = str(tmp_path / "nccl_jni_shim.o")
    cmd = ["g++", "-std=c++17", "-c", "-fPIC", "-fvisibility=hidden", "-DBIDMAT_B200_WITH_JNI=1",
           "-DBIDMAT_B200_WITH_NCCL=1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "tests", "jni_stub"),
           "-I", os.path.dirname(nccl), "-I", os.path.dirname(cuda),
           os.path.join(ROOT, "bidmat_b200", "csrc", "nccl_jni_shim.cpp"), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    syms = subprocess.run(["nm", "-g", "--defined-only", obj], capture_output=True, text=True).stdout
    for name in ("hasNCCL", "ncclCommInitAll", "ncclCommDestroy", "ncclAllReduce"):
        assert ("Java_edu_berkeley_bid_NCCL_" + name + "\n") in syms, name
    undefined = subprocess.run(["nm", "-u", obj], capture_output=True, text=True).stdout
    for name in ("ncclGroupStart", "ncclGroupEnd", "ncclAllReduce", "ncclCommInitAll"):
        assert name in undefined, name


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_matkernel_launcher_symbols(tmp_path):
    """The C++ launcher names of jni/include/MatKernel.hpp:47-53,140-156 and MatKernelD.hpp:43-55,
    with their exact argument lists, so that BIDMat's own JNI glue links against them unchanged."""
    obj = str(tmp_path / "matkernel_compat.o")
    cmd = ["g++", "-std=c++17", "-c", "-fPIC", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "bidmat_b200", "csrc", "matkernel_compat.cpp"), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    syms = subprocess.run(["nm", "-C", "--defined-only", obj], capture_output=True, text=True).stdout
    for sig in ("dsmult(int, int, int, float*, float*, int*, int*, float*)",
                "dsmultT(int, int, int, float*, float*, int*, int*, float*)",
                "dds(int, int, float*, float*, int*, int*, float*)",
                "dds0(int, int, float*, float*, int*, int*, float*)",
                "dsmult_tune(int, int, int, float*, float*, int*, int*, float*, int, int)",
                "dsmultx_tune(int, int, int, float*, float*, int*, int*, float*, int, int, int)",
                "dsmultTile(int, int, int, int, float*, int, float*, int*, int*, int, int, float*, int)",
                "dsmultTileT(int, int, int, int, float*, int, float*, int*, int*, int, int, float*, int)",
                "spsum(int, int, int, int*, int*, float*, float*, int)",
                "sdoprow(int, int, int, float*, int*, float*, int, int)",
                "sdopcol(int, int, int, float*, int*, float*, int, int)",
                "dsmult(int, int, int, double*, double*, int*, int*, double*)",
                "dsmultT(int, int, int, double*, double*, int*, int*, double*)",
                "dds(int, int, double*, double*, int*, int*, double*)",
                "dds0(int, int, double*, double*, int*, int*, double*)",
                "spsum(int, int, int, int*, int*, double*, double*, int)",
                "sdoprow(int, int, int, double*, int*, double*, int, int)",
                "sdopcol(int, int, int, double*, int*, double*, int, int)"):
        assert (" T " + sig + "\n") in syms, sig
    undefined = subprocess.run(["nm", "-u", obj], capture_output=True, text=True).stdout
    from bidmat_b200 import _lib
    declared = set(_lib.declared_symbols())
    called = [line.split()[-1] for line in undefined.splitlines() if "bidmat_b200_" in line]
    assert called and all(sym in declared for sym in called), called
