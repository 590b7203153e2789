"""The shared library loads without a GPU and exports exactly what the public
header declares; the product has no CPU fallback."""
import ctypes
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_builds_and_exports_every_declared_symbol():
    from bidmat_b200 import build
    path = build.build()
    assert os.path.exists(path)
    from bidmat_b200 import _lib
    declared = _lib.declared_symbols()
    assert len(declared) >= 18
    lib = ctypes.CDLL(path)
    for name in declared:
        assert hasattr(lib, name), "header declares %s but the library does not export it" % name
    assert set(declared) == set(_lib._SIGNATURES), "ctypes signatures and header drifted apart"
    assert lib.bidmat_b200_version() >= 100
    assert lib.bidmat_b200_launch_count() == 0


def test_header_cites_the_reference_interface_for_each_replacement():
    text = open(os.path.join(ROOT, "include", "bidmat_b200.h")).read()
    for cite in ("MatKernel.hpp:140", "MatKernel.hpp:150", "MatKernel.hpp:154", "MatKernel.hpp:156",
                 "CUMAT.java:143", "CUMAT.java:152", "CUMAT.java:211", "CUMAT.java:213",
                 "BIDMat_CUMAT.cpp:722", "BIDMat_CUMAT.cpp:761", "BIDMat_CUMAT.cpp:774", "BIDMat_CUMAT.cpp:787"):
        assert cite in text, cite


def test_argument_validation_needs_no_device():
    """Size checks and the nnz == 0 no-op are decided on the host before any
    CUDA call, so they can be exercised without a GPU."""
    from bidmat_b200 import _lib
    L = _lib.lib
    assert L.bidmat_b200_dsmult(4, 4, 0, 0, 0, 0, 0, 0) == 0
    assert L.bidmat_b200_dsmultT(4, 4, 0, 0, 0, 0, 0, 0) == 0
    assert L.bidmat_b200_dds(4, 0, 0, 0, 0, 0, 0) == 0
    assert L.bidmat_b200_dsmult_async(-1, 4, 4, 0, 0, 0, 0, 0, 0) == 1      # cudaErrorInvalidValue
    assert L.bidmat_b200_dsmult_async(4, 4, 4, 0, 0, 0, 0, 0, 0) == 1       # null pointers
    assert L.bidmat_b200_dds_async(4, -2, 0, 0, 0, 0, 0, 0) == 1
    assert _lib.error_string(1)


def test_product_modules_never_import_the_oracle():
    pkg = os.path.join(ROOT, "bidmat_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f
                assert "liboracle" not in src and "oracle/" not in src, f


def test_missing_library_fails_loudly():
    code = ("import bidmat_b200._lib as L\n"
            "try:\n    L.load('/nonexistent/libbidmatcuda_b200.so')\n"
            "except ImportError as e:\n    print('OK', 'no CPU fallback' in str(e))\n")
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert "OK True" in out.stdout, out.stdout + out.stderr
