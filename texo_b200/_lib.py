"""ctypes binding of libtexo_b200.so (the combined C-ABI library).

There is no CPU fallback: if the library is missing it is built with nvcc, and if that is
impossible the import of the operators fails with an error.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

_LIB = None

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_ptr = ctypes.c_void_p

_SIGNATURES = {
    # name: (restype, argtypes)
    "texo_mm_int8_solve": (None, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                  _c_float, _c_float, _c_float, _c_int, _c_int, _c_int]),
    "texo_mm_int8_solve_per_channel": (None, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                              _c_float, _c_ptr, _c_float, _c_int, _c_ptr, _c_int]),
    "texo_mm_int8_solve_per_group": (None, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                            _c_float, _c_ptr, _c_float, _c_int, _c_int, _c_int]),
    "texo_mm_int4a8_solve_per_group": (None, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                              _c_float, _c_ptr, _c_float, _c_int, _c_int, _c_int]),
    "texo_set_sums_epoch": (None, [ctypes.c_uint]),
    "texo_mm_int8_swiglu_solve": (None, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                         _c_float, _c_float, _c_float, _c_float,
                                         _c_int, _c_int, _c_int, _c_int]),
    "texo_mm_int8_dequant_solve": (None, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                          _c_float, _c_float, _c_int, _c_int]),
    "texo_mm_int8_solve_allgather": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                             _c_int, _c_int, _c_float, _c_float, _c_float,
                                             _c_int, _c_int, _c_int]),
    "texo_mm_int8_solve_allgather_multicast": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                                                        _c_int, _c_int, _c_int, _c_int, _c_float,
                                                        _c_float, _c_float, _c_int, _c_int, _c_int]),
    "texo_mm_int8_solve_noalloc": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                            _c_float, _c_float, _c_float, _c_int, _c_int, _c_int]),
    "texo_mm_int8_noalloc_status": (_c_int, []),
    "texo_mm_int8_solve_host": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                         _c_float, _c_float, _c_float, _c_int, _c_int, _c_int]),
    "texo_mm_int8_prepare_weights": (_c_ptr, [_c_ptr, _c_int, _c_int]),
    "texo_mm_int8_release_weights": (None, [_c_ptr]),
    "texo_mm_int8_solve_prepared": (None, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_float, _c_float, _c_float,
                                           _c_int, _c_int, _c_int]),
    "texo_mm_int4_solve": (None, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int]),
    "texo_dequantization_solve": (None, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int]),
    "texo_mm_int4a8_solve": (None, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                    _c_float, _c_float, _c_float, _c_int, _c_int, _c_int]),
    "texo_mm_int4a8_solve_per_channel": (None, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                                _c_float, _c_ptr, _c_float, _c_int, _c_ptr, _c_int]),
    "texo_rms_norm_w_residual_solve": (None, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_float]),
    "texo_rms_norm_quant_solve": (None, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                                         _c_float, _c_float, _c_int]),
    "texo_mm_int8_solve_presummed": (None, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_float, _c_float,
                                            _c_float, _c_int, _c_int, _c_int]),
    "texo_rms_norm_last_path": (_c_int, []),
    "texo_mm_int4a8_last_path": (_c_int, []),
    "texo_mm_int4a8_force_path": (None, [_c_int]),
    "texo_mm_int4a8_status": (_c_int, []),
    "texo_mm_int8_last_path": (_c_int, []),
    "texo_mm_int8_force_path": (None, [_c_int]),
    "texo_mm_int8_status": (_c_int, []),
    "texo_mm_int4_last_path": (_c_int, []),
    "texo_mm_int4_force_path": (None, [_c_int]),
    "texo_mm_int4_status": (_c_int, []),
    "texo_selftest_wait_timeout": (_c_int, []),
    "texo_kernel_launches": (ctypes.c_longlong, []),
    "texo_tensor_map_cache_stats": (None, [ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong)]),
    "texo_profile_enable": (None, [_c_int]),
    "texo_int8_issue_ceiling_tops": (ctypes.c_double, [_c_int, _c_int]),
    "texo_int8_issue_rate_tops": (ctypes.c_double, [_c_int, _c_int, _c_int]),
    "texo_f16_issue_rate_tflops": (ctypes.c_double, [_c_int, _c_int, _c_int]),
    "texo_int8_feed_rate_tbs": (ctypes.c_double, [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int]),
    "texo_profile_read": (_c_int, [ctypes.POINTER(_c_float), ctypes.POINTER(_c_int)]),
}


def library_path() -> str:
    return _build.lib_path("texo_b200")


def load() -> ctypes.CDLL:
    """Load (building first if needed) the combined library; raises if unavailable."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        _build.build()
    if not os.path.exists(path):
        raise RuntimeError(f"texo_b200: CUDA library {path} is missing and could not be built")
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means a stale or foreign library
        fn.restype = restype
        fn.argtypes = argtypes
    _LIB = lib
    return lib
