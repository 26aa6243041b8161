"""ctypes binding of the CUDA library.  There is no fallback: if the library is missing or does not
load, importing this module raises."""

from __future__ import annotations

import ctypes
import os

from . import _build

_LIB = None


def lib() -> ctypes.CDLL:
    """Load (once) ``_lib/liblethe_gdn.so``.  The library is built by ``_build.build()``; a missing
    file is an error, never a reason to compute elsewhere."""
    global _LIB
    if _LIB is None:
        path = _build.LIB
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m lethe_b200._build` (needs nvcc)")
        _LIB = ctypes.CDLL(path)
        _declare(_LIB)
    return _LIB


def _declare(L: ctypes.CDLL) -> None:
    c_int, c_void_p = ctypes.c_int, ctypes.c_void_p
    L.lethe_gdn_saved_bytes.restype = ctypes.c_size_t
    L.lethe_gdn_saved_bytes.argtypes = [c_void_p]
    L.lethe_gdn_scratch_bytes.restype = ctypes.c_size_t
    L.lethe_gdn_scratch_bytes.argtypes = [c_void_p]
    L.lethe_gdn_forward.restype = c_int
    L.lethe_gdn_forward.argtypes = [c_void_p, c_void_p]
    L.lethe_gdn_backward.restype = c_int
    L.lethe_gdn_backward.argtypes = [c_void_p, c_void_p]
    L.lethe_gdn_forward_static.restype = c_int
    L.lethe_gdn_forward_static.argtypes = [c_void_p, c_void_p]
    L.lethe_gdn_forward_static_capacity.restype = ctypes.c_size_t
    L.lethe_gdn_forward_static_capacity.argtypes = []
    L.lethe_gdn_decode_step.restype = c_int
    L.lethe_gdn_decode_step.argtypes = [c_void_p, c_void_p]
    L.lethe_gdn_l2norm_qk.restype = c_int
    L.lethe_gdn_l2norm_qk.argtypes = [c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32,
                                                      ctypes.c_float, c_void_p]
    L.lethe_gdn_l2norm_qk_vjp.restype = c_int
    L.lethe_gdn_l2norm_qk_vjp.argtypes = [c_void_p] * 6 + [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32,
                                                          ctypes.c_float, c_void_p]
    L.lethe_gdn_strerror.restype = ctypes.c_char_p
    L.lethe_gdn_strerror.argtypes = [c_int]
