"""ctypes binding of the C ABI in include/bidmat_b200.h.

There is no CPU fallback: when the shared library is missing or a symbol
declared in the header is not exported, importing this module raises.
"""
import ctypes
import os
import re

_PKG = os.path.dirname(os.path.abspath(__file__))
LIBPATH = os.path.join(_PKG, "lib", "libbidmatcuda_b200.so")
HEADER = os.path.join(_PKG, "..", "include", "bidmat_b200.h")

_c_int = ctypes.c_int
_vp = ctypes.c_void_p

# name -> (restype, argtypes); pointers travel as integers (device addresses).
_SIGNATURES = {
    "bidmat_b200_dsmult": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dsmultT": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dds": (_c_int, [_c_int, _c_int, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dds0": (_c_int, [_c_int, _c_int, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dsmult_tune": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _c_int, _c_int]),
    "bidmat_b200_dsmultx_tune": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _c_int, _c_int, _c_int]),
    "bidmat_b200_dsmult_async": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dsmultT_async": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _c_int, _vp]),
    "bidmat_b200_dsmult_f64": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dsmultT_f64": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dds_f64": (_c_int, [_c_int, _c_int, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dds0_f64": (_c_int, [_c_int, _c_int, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dsmult_f64_async": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dsmultT_f64_async": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _c_int, _vp]),
    "bidmat_b200_dds_f64_async": (_c_int, [_c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dsmultT_plan_create": (_c_int, [_c_int, _c_int, _c_int, _c_int, _vp, _vp, _c_int, _vp,
                                                 ctypes.POINTER(_vp)]),
    "bidmat_b200_dsmultT_planned": (_c_int, [_vp, _c_int, _c_int, _c_int, _vp, _vp, _vp, _c_int, _vp]),
    "bidmat_b200_dsmultT_planned_f64": (_c_int, [_vp, _c_int, _c_int, _c_int, _vp, _vp, _vp, _c_int, _vp]),
    "bidmat_b200_plan_verify": (_c_int, [_vp, _c_int, _c_int, _vp, _vp, _vp]),
    "bidmat_b200_plan_info": (_c_int, [_vp, ctypes.POINTER(ctypes.c_longlong), _c_int]),
    "bidmat_b200_plan_touched_rows": (_c_int, [_vp, _vp, _vp]),
    "bidmat_b200_plan_destroy": (_c_int, [_vp]),
    "bidmat_b200_set_workspace_limit": (_c_int, [ctypes.c_longlong]),
    "bidmat_b200_set_auto_plan": (_c_int, [_c_int]),
    "bidmat_b200_auto_plan_info": (_c_int, [ctypes.POINTER(ctypes.c_longlong), _c_int]),
    "bidmat_b200_dsmult_noalloc": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dds_async": (_c_int, [_c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dsmult_dds_async": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dds0_async": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_peer_allreduce_sum": (_c_int, [_c_int, _c_int, ctypes.POINTER(ctypes.c_ulonglong),
                                                ctypes.c_longlong, _c_int, _vp]),
    "bidmat_b200_peer_allreduce_sum_rows": (_c_int, [_c_int, _c_int, ctypes.POINTER(ctypes.c_ulonglong), _c_int,
                                                     ctypes.c_longlong, _vp, _c_int, _vp]),
    "bidmat_b200_mc_allreduce_sum": (_c_int, [_c_int, _c_int, _vp, ctypes.c_longlong, _c_int, _vp]),
    "bidmat_b200_mc_allreduce_sum_range": (_c_int, [_c_int, _c_int, _vp, ctypes.c_longlong, ctypes.c_longlong, _c_int,
                                                    _vp]),
    "bidmat_b200_plan_clear_untouched": (_c_int, [_vp, _c_int, _vp, _vp]),
    "bidmat_b200_peer_allreduce_sum_rows_range": (_c_int, [_c_int, _c_int, ctypes.POINTER(ctypes.c_ulonglong), _c_int,
                                                           ctypes.c_longlong, _vp, ctypes.c_longlong, ctypes.c_longlong,
                                                           _c_int, _vp]),
    "bidmat_b200_plan_row_parts": (_c_int, [_vp, _c_int, ctypes.POINTER(_c_int)]),
    "bidmat_b200_dsmultT_planned_part": (_c_int, [_vp, _c_int, _c_int, _c_int, _vp, _vp, _vp, _c_int, _c_int, _vp]),
    "bidmat_b200_expand_jc": (_c_int, [_c_int, _c_int, _vp, _vp, _vp]),
    "bidmat_b200_compress_ic": (_c_int, [_c_int, _c_int, _vp, _vp, _vp]),
    "bidmat_b200_transpose_csc": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bidmat_b200_dsmultTile": (_c_int, [_c_int, _c_int, _c_int, _c_int, _vp, _c_int, _vp, _vp, _vp, _c_int, _c_int,
                                        _vp, _c_int, _c_int]),
    "bidmat_b200_sdoprow": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _c_int, _c_int]),
    "bidmat_b200_sdopcol": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _c_int, _c_int]),
    "bidmat_b200_spsum": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _c_int]),
    "bidmat_b200_spsum_f64": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _vp, _c_int]),
    "bidmat_b200_sdoprow_f64": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _c_int, _c_int]),
    "bidmat_b200_sdopcol_f64": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp, _vp, _c_int, _c_int]),
    "bidmat_b200_check_structure": (_c_int, [_c_int, _c_int, _c_int, _vp, _vp]),
    "bidmat_b200_workspace_bytes": (ctypes.c_longlong, []),
    "bidmat_b200_release_workspace": (_c_int, []),
    "bidmat_b200_launch_count": (ctypes.c_longlong, []),
    "bidmat_b200_timing_enable": (_c_int, [_c_int]),
    "bidmat_b200_timing_read": (_c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_double),
                                         ctypes.POINTER(ctypes.c_longlong)]),
    "bidmat_b200_timing_reset": (_c_int, []),
    "bidmat_b200_version": (_c_int, []),
    "bidmat_b200_error_string": (ctypes.c_char_p, [_c_int]),
}


def declared_symbols(header=HEADER):
    """Names of the functions the public header declares."""
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bidmat_b200_[A-Za-z0-9_]+)\s*\(", text)))


def load(path=LIBPATH):
    if not os.path.exists(path):
        raise ImportError(
            "%s is missing: build it with `python -m bidmat_b200.build` "
            "(there is no CPU fallback for this library)" % path)
    lib = ctypes.CDLL(path)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load()


def error_string(err):
    return lib.bidmat_b200_error_string(int(err)).decode()


def timing_read(label):
    """(total milliseconds, number of launches) recorded under `label`."""
    ms = ctypes.c_double(0.0)
    cnt = ctypes.c_longlong(0)
    err = lib.bidmat_b200_timing_read(label.encode(), ctypes.byref(ms), ctypes.byref(cnt))
    if err != 0:
        raise RuntimeError("timing_read: " + error_string(err))
    return ms.value, cnt.value
