"""ctypes front end of the CPU checker (TEST INFRASTRUCTURE, not product code).

Conventions: dense matrices are numpy float32 arrays of shape (ncols, k), C
contiguous, which is BIDMat's column-major k x ncols layout
(src/main/scala/BIDMat/FMat.scala data array); S is CSC with 0-based int32
``jc`` (n+1), ``ir`` (nnz) and float32 ``data`` (nnz).

dsmult / dsmultT ACCUMULATE into the array passed as ``out`` (FMat.madd /
FMat.maddT semantics, FMat.scala:1167, 1410); when ``out`` is None a zeroed
array is used, which is what ``A * S`` and ``B *^ S`` do (FMat.scala:1162,
1405).  dds STORES (MatFunctions.scala:1612).
"""
import ctypes
import os

import numpy as np

from . import build as _build

_F32P = ctypes.POINTER(ctypes.c_float)
_F64P = ctypes.POINTER(ctypes.c_double)
_I32P = ctypes.POINTER(ctypes.c_int32)

_lib = None
_libs = {}
_ref = None
_ref_tried = False
_ref_gpu = None
_ref_gpu_tried = False
_variant = "plain"


def use_native(on=True):
    """Selects which build of spdense_oracle.c the functions below call: the plain
    x86-64 build (default) or the -O3 -march=native build made on this machine.
    Both give the same bits (contraction is off in both); the native one is what
    the benchmark times.  Returns the variant actually in use."""
    global _variant, _lib
    want = "native" if on else "plain"
    if want == "native" and _build.build_oracle_native() is None:
        want = "plain"
    _variant = want
    _lib = None
    return want


def _load():
    global _lib
    if _lib is None and _variant in _libs:
        _lib = _libs[_variant]
    if _lib is None:
        _lib = ctypes.CDLL(_build.build_oracle_native() if _variant == "native" else _build.build_oracle())
        _libs[_variant] = _lib
        for name in ("oracle_dsmult", "oracle_dsmultT"):
            getattr(_lib, name).argtypes = [ctypes.c_int, ctypes.c_int, _F32P, _F32P, _I32P, _I32P,
                                            _F32P, ctypes.c_int]
            getattr(_lib, name).restype = None
        _lib.oracle_dds.argtypes = [ctypes.c_int, ctypes.c_int, _F32P, _F32P, _I32P, _I32P, _F32P,
                                    ctypes.c_int]
        _lib.oracle_dds.restype = None
        for name in ("oracle_dsmult_f64", "oracle_dsmultT_f64"):
            getattr(_lib, name).argtypes = [ctypes.c_int, ctypes.c_int, _F32P, _F32P, _I32P, _I32P,
                                            _F64P, _F64P, ctypes.c_int]
            getattr(_lib, name).restype = None
        _lib.oracle_dds_f64.argtypes = [ctypes.c_int, ctypes.c_int, _F32P, _F32P, _I32P, _I32P,
                                        _F64P, _F64P, ctypes.c_int]
        _lib.oracle_dds_f64.restype = None
        for name in ("oracle_dsmultT_d", "oracle_dds_d"):
            getattr(_lib, name).restype = None
        _lib.oracle_dsmult_d.argtypes = [ctypes.c_int, ctypes.c_int, _F64P, _F64P, _I32P, _I32P, _F64P, ctypes.c_int]
        _lib.oracle_dsmult_d.restype = None
        _lib.oracle_dsmultT_d.argtypes = [ctypes.c_int, ctypes.c_int, _F64P, _F64P, _I32P, _I32P, _F64P]
        _lib.oracle_dds_d.argtypes = [ctypes.c_int, ctypes.c_int, _F64P, _F64P, _I32P, _I32P, _F64P]
        _lib.oracle_uncompress_inds.argtypes = [_I32P, ctypes.c_int, _I32P]
        _lib.oracle_uncompress_inds.restype = None
        _lib.oracle_compress_inds.argtypes = [_I32P, ctypes.c_int, ctypes.c_int32, _I32P]
        _lib.oracle_compress_inds.restype = None
        _lib.oracle_check_csc.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int32, _I32P, _I32P]
        _lib.oracle_check_csc.restype = ctypes.c_int
    return _lib


def _load_ref():
    global _ref, _ref_tried
    if not _ref_tried:
        _ref_tried = True
        path = _build.build_reference()
        if path and os.path.exists(path):
            _ref = ctypes.CDLL(path)
            for name in ("ref_smcscm", "ref_smcsrm"):
                getattr(_ref, name).argtypes = [ctypes.c_int, ctypes.c_int, _F32P, _F32P, _I32P,
                                                _I32P, _F32P]
                getattr(_ref, name).restype = None
            for name in ("ref_dmcscm", "ref_dmcsrm"):
                getattr(_ref, name).argtypes = [ctypes.c_int, ctypes.c_int, _F64P, _F64P, _I32P,
                                                _I32P, _F64P]
                getattr(_ref, name).restype = None
    return _ref


def default_threads():
    return os.cpu_count() or 1


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_F32P)


def _i32(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(_I32P)


def _dense_k(a):
    if a.ndim != 2:
        raise ValueError("dense operand must be 2-D (ncols, k)")
    return int(a.shape[1])


def dsmult(A, data, ir, jc, out=None, nthreads=None):
    """C(k x n) += A(k x m) * S.  FMat.fSMultHelper order."""
    A, pA = _f32(A)
    k = _dense_k(A)
    data, pd = _f32(data)
    ir, pir = _i32(ir)
    jc, pjc = _i32(jc)
    n = len(jc) - 1
    if out is None:
        out = np.zeros((n, k), dtype=np.float32)
    assert out.dtype == np.float32 and out.flags.c_contiguous and out.shape == (n, k)
    _load().oracle_dsmult(k, n, pA, pd, pir, pjc, out.ctypes.data_as(_F32P),
                          nthreads or default_threads())
    return out


def dsmultT(B, data, ir, jc, m, out=None, nthreads=None):
    """C(k x m) += B(k x n) * S^T.  FMat.fSMultTHelper2 order."""
    B, pB = _f32(B)
    k = _dense_k(B)
    data, pd = _f32(data)
    ir, pir = _i32(ir)
    jc, pjc = _i32(jc)
    n = len(jc) - 1
    assert B.shape[0] == n
    if out is None:
        out = np.zeros((m, k), dtype=np.float32)
    assert out.dtype == np.float32 and out.flags.c_contiguous and out.shape == (m, k)
    _load().oracle_dsmultT(k, n, pB, pd, pir, pjc, out.ctypes.data_as(_F32P),
                           nthreads or default_threads())
    return out


def dds(A, B, ir, jc, nthreads=None):
    """P.data[j] = <A[:, ir[j]], B[:, col(j)]>.  MatFunctions.DDShelper order."""
    A, pA = _f32(A)
    B, pB = _f32(B)
    k = _dense_k(A)
    assert _dense_k(B) == k
    ir, pir = _i32(ir)
    jc, pjc = _i32(jc)
    n = len(jc) - 1
    out = np.zeros(len(ir), dtype=np.float32)
    _load().oracle_dds(k, n, pA, pB, pir, pjc, out.ctypes.data_as(_F32P),
                       nthreads or default_threads())
    return out


def dsmult_f64(A, data, ir, jc, nthreads=None):
    """fp64 value and sum|term| of A*S."""
    A, pA = _f32(A)
    k = _dense_k(A)
    data, pd = _f32(data)
    ir, pir = _i32(ir)
    jc, pjc = _i32(jc)
    n = len(jc) - 1
    out = np.zeros((n, k), dtype=np.float64)
    oab = np.zeros((n, k), dtype=np.float64)
    _load().oracle_dsmult_f64(k, n, pA, pd, pir, pjc, out.ctypes.data_as(_F64P),
                              oab.ctypes.data_as(_F64P), nthreads or default_threads())
    return out, oab


def dsmultT_f64(B, data, ir, jc, m, nthreads=None):
    """fp64 value and sum|term| of B*^S."""
    B, pB = _f32(B)
    k = _dense_k(B)
    data, pd = _f32(data)
    ir, pir = _i32(ir)
    jc, pjc = _i32(jc)
    n = len(jc) - 1
    out = np.zeros((m, k), dtype=np.float64)
    oab = np.zeros((m, k), dtype=np.float64)
    _load().oracle_dsmultT_f64(k, n, pB, pd, pir, pjc, out.ctypes.data_as(_F64P),
                               oab.ctypes.data_as(_F64P), nthreads or default_threads())
    return out, oab


def dds_f64(A, B, ir, jc, nthreads=None):
    """fp64 value and sum|term| of DDS."""
    A, pA = _f32(A)
    B, pB = _f32(B)
    k = _dense_k(A)
    ir, pir = _i32(ir)
    jc, pjc = _i32(jc)
    n = len(jc) - 1
    out = np.zeros(len(ir), dtype=np.float64)
    oab = np.zeros(len(ir), dtype=np.float64)
    _load().oracle_dds_f64(k, n, pA, pB, pir, pjc, out.ctypes.data_as(_F64P),
                           oab.ctypes.data_as(_F64P), nthreads or default_threads())
    return out, oab


def uncompress_inds(jc):
    jc, pjc = _i32(jc)
    n = len(jc) - 1
    ic = np.empty(int(jc[n]), dtype=np.int32)
    _load().oracle_uncompress_inds(pjc, n, ic.ctypes.data_as(_I32P))
    return ic


def compress_inds(ic, n):
    ic, pic = _i32(ic)
    jc = np.empty(n + 1, dtype=np.int32)
    _load().oracle_compress_inds(pic, n, len(ic), jc.ctypes.data_as(_I32P))
    return jc


def check_csc(m, n, ir, jc):
    ir, pir = _i32(ir)
    jc, pjc = _i32(jc)
    return _load().oracle_check_csc(m, n, len(ir), pir, pjc)


def ref_available():
    return _load_ref() is not None


def ref_smcscm(A, data, ir, jc, out=None):
    """The reference's own compiled loop for A*S (BIDMat_SPBLAS.c:364-395).
    Uses OpenMP's default thread count over columns, as the reference does."""
    lib = _load_ref()
    if lib is None:
        raise RuntimeError("reference build oracle/_ref/libspblas_ref.so is not available")
    A, pA = _f32(A)
    k = _dense_k(A)
    data, pd = _f32(data)
    ir, pir = _i32(ir)
    jc, pjc = _i32(jc)
    n = len(jc) - 1
    if out is None:
        out = np.zeros((n, k), dtype=np.float32)
    lib.ref_smcscm(k, n, pA, pd, pir, pjc, out.ctypes.data_as(_F32P))
    return out


def ref_smcsrm(B, data, ir, jc, m, out=None):
    """The reference's own compiled loop for B*^S (BIDMat_SPBLAS.c:397-427);
    single-threaded, as in the reference."""
    lib = _load_ref()
    if lib is None:
        raise RuntimeError("reference build oracle/_ref/libspblas_ref.so is not available")
    B, pB = _f32(B)
    k = _dense_k(B)
    data, pd = _f32(data)
    ir, pir = _i32(ir)
    jc, pjc = _i32(jc)
    n = len(jc) - 1
    if out is None:
        out = np.zeros((m, k), dtype=np.float32)
    lib.ref_smcsrm(k, n, pB, pd, pir, pjc, out.ctypes.data_as(_F32P))
    return out


# ---- double-precision operands (BIDMat's DMat / SDMat path)
def _f64(a):
    a = np.ascontiguousarray(a, dtype=np.float64)
    return a, a.ctypes.data_as(_F64P)


def dsmult_d(A, data, ir, jc, out=None, nthreads=None):
    A, pA = _f64(A); k = _dense_k(A); data, pd = _f64(data); ir, pir = _i32(ir); jc, pjc = _i32(jc)
    n = len(jc) - 1
    if out is None:
        out = np.zeros((n, k), dtype=np.float64)
    _load().oracle_dsmult_d(k, n, pA, pd, pir, pjc, out.ctypes.data_as(_F64P), nthreads or default_threads())
    return out


def dsmultT_d(B, data, ir, jc, m, out=None):
    B, pB = _f64(B); k = _dense_k(B); data, pd = _f64(data); ir, pir = _i32(ir); jc, pjc = _i32(jc)
    n = len(jc) - 1
    if out is None:
        out = np.zeros((m, k), dtype=np.float64)
    _load().oracle_dsmultT_d(k, n, pB, pd, pir, pjc, out.ctypes.data_as(_F64P))
    return out


def dds_d(A, B, ir, jc):
    A, pA = _f64(A); B, pB = _f64(B); k = _dense_k(A); ir, pir = _i32(ir); jc, pjc = _i32(jc)
    n = len(jc) - 1
    out = np.zeros(len(ir), dtype=np.float64)
    _load().oracle_dds_d(k, n, pA, pB, pir, pjc, out.ctypes.data_as(_F64P))
    return out


def ref_dmcscm(A, data, ir, jc, out=None):
    lib = _load_ref()
    if lib is None:
        raise RuntimeError("reference build oracle/_ref/libspblas_ref.so is not available")
    A, pA = _f64(A); k = _dense_k(A); data, pd = _f64(data); ir, pir = _i32(ir); jc, pjc = _i32(jc)
    n = len(jc) - 1
    if out is None:
        out = np.zeros((n, k), dtype=np.float64)
    lib.ref_dmcscm(k, n, pA, pd, pir, pjc, out.ctypes.data_as(_F64P))
    return out


def ref_dmcsrm(B, data, ir, jc, m, out=None):
    lib = _load_ref()
    if lib is None:
        raise RuntimeError("reference build oracle/_ref/libspblas_ref.so is not available")
    B, pB = _f64(B); k = _dense_k(B); data, pd = _f64(data); ir, pir = _i32(ir); jc, pjc = _i32(jc)
    n = len(jc) - 1
    if out is None:
        out = np.zeros((m, k), dtype=np.float64)
    lib.ref_dmcsrm(k, n, pB, pd, pir, pjc, out.ctypes.data_as(_F64P))
    return out


# ---- the reference's own CUDA launchers (jni/src/Arith.cu), compiled for sm_100a.
# Arguments are device addresses as integers; each call synchronises the legacy
# default stream and returns a cudaError_t (0 = success), as the launchers do.
def _load_ref_gpu():
    global _ref_gpu, _ref_gpu_tried
    if not _ref_gpu_tried:
        _ref_gpu_tried = True
        path = _build.build_reference_gpu()
        if path and os.path.exists(path):
            vp, ci = ctypes.c_void_p, ctypes.c_int
            _ref_gpu = ctypes.CDLL(path)
            _ref_gpu.ref_gpu_dsmult.argtypes = [ci, ci, ci, vp, vp, vp, vp, vp]
            _ref_gpu.ref_gpu_dsmultT.argtypes = [ci, ci, ci, vp, vp, vp, vp, vp]
            _ref_gpu.ref_gpu_dds.argtypes = [ci, ci, vp, vp, vp, vp, vp]
            _ref_gpu.ref_gpu_dds0.argtypes = [ci, ci, vp, vp, vp, vp, vp]
            _ref_gpu.ref_gpu_spsum.argtypes = [ci, ci, ci, vp, vp, vp, vp, ci]
            for name in ("ref_gpu_dsmult", "ref_gpu_dsmultT", "ref_gpu_dds", "ref_gpu_dds0", "ref_gpu_spsum"):
                getattr(_ref_gpu, name).restype = ci
    return _ref_gpu


def ref_gpu_available():
    return _load_ref_gpu() is not None


def _ref_gpu_call(name, *args):
    lib = _load_ref_gpu()
    if lib is None:
        raise RuntimeError("reference build oracle/_ref/libarith_ref.so is not available")
    err = getattr(lib, name)(*args)
    if err != 0:
        raise RuntimeError("%s returned CUDA error %d" % (name, err))


def ref_gpu_dsmult(k, n, nnz, A, data, ir, ic, C):
    """dsmult (jni/src/Arith.cu:46-60): C += A * S, float atomics."""
    _ref_gpu_call("ref_gpu_dsmult", k, n, nnz, A, data, ir, ic, C)


def ref_gpu_dsmultT(k, n, nnz, B, data, ir, ic, C):
    """dsmultT (jni/src/Arith.cu:234-248): C += B * S^T, float atomics."""
    _ref_gpu_call("ref_gpu_dsmultT", k, n, nnz, B, data, ir, ic, C)


def ref_gpu_dds(k, nnz, A, B, ir, ic, P):
    """dds (jni/src/Arith.cu:381-389): P[j] += <A[:, ir[j]], B[:, ic[j]]>."""
    _ref_gpu_call("ref_gpu_dds", k, nnz, A, B, ir, ic, P)


def ref_gpu_dds0(k, n, A, B, ir, jc, P):
    """dds0 (jni/src/Arith.cu:391-399); k must be 1024."""
    _ref_gpu_call("ref_gpu_dds0", k, n, A, B, ir, jc, P)


def ref_gpu_spsum(m, n, nnz, ir, ic, P, B, which):
    """spsum (jni/src/Arith.cu:267-277): which == 1 column sums, else row sums."""
    _ref_gpu_call("ref_gpu_spsum", m, n, nnz, ir, ic, P, B, which)
