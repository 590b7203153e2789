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
