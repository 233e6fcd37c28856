"""ctypes binding of ``libcats_b200.so`` (the C ABI declared in ``include/cats_b200.h``).

There is no CPU or PyTorch fallback: if the shared object cannot be loaded, every operator of
this package raises.  Use :func:`lib` to get the loaded library and :func:`check` to turn a
status code into a ``RuntimeError``.
"""
from __future__ import annotations

import ctypes
import os
import threading

from . import _build

F32, F16, BF16 = 0, 1, 2
OUT_STORE, OUT_ACC_F32 = 0, 1
# status codes of include/cats_b200.h
OK, ERR_DTYPE, ERR_SHAPE, ERR_ALIGN, ERR_NULL = 0, -1, -2, -3, -4
ERR_WORKSPACE, ERR_CUDA, ERR_MODE, ERR_STATIC_LIMIT = -5, -6, -7, -8
MAX_BATCH = 16

_c_void_p = ctypes.c_void_p
_c_int = ctypes.c_int
_c_size_t = ctypes.c_size_t
_c_float = ctypes.c_float

# name -> (restype, argtypes); mirrors include/cats_b200.h one to one
SIGNATURES = {
    "cats_abi_version": (_c_int, []),
    "cats_status_string": (ctypes.c_char_p, [_c_int]),
    "cats_last_cuda_error": (ctypes.c_char_p, []),
    "cats_sm_count": (_c_int, []),
    "cats_set_option": (_c_int, [ctypes.c_char_p, _c_int]),
    "cats_workspace_bytes": (_c_size_t, [_c_int, _c_int, _c_int]),
    "cats_workspace_init": (_c_int, [_c_void_p, _c_size_t, _c_void_p]),
    "cats_gate": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_size_t, _c_int, _c_int, _c_int,
                           _c_int, _c_float, _c_void_p, _c_void_p, _c_void_p]),
    "cats_compact": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_size_t, _c_int, _c_int, _c_int,
                              _c_int, _c_float, _c_void_p]),
    "cats_up": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_size_t, _c_int, _c_int, _c_int,
                         _c_int, _c_void_p, _c_void_p]),
    "cats_down": (_c_int, [_c_void_p, _c_void_p, _c_size_t, _c_int, _c_int, _c_int, _c_int,
                           _c_void_p, _c_int, _c_void_p]),
    "cats_updown": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t, _c_int,
                             _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                             _c_void_p, _c_float, _c_void_p]),
    "cats_mlp": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t,
                          _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_int, _c_void_p,
                          _c_void_p, _c_void_p, _c_float, _c_void_p]),
    "cats_mlp_dense": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t,
                                _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_int, _c_void_p,
                                _c_void_p, _c_void_p, _c_float, _c_void_p]),
    "cats_dense_supported": (_c_int, [_c_int, _c_int, _c_int, _c_int]),
    "cats_mlp_stack_dense": (_c_int, [_c_int, ctypes.POINTER(_c_void_p), ctypes.POINTER(_c_void_p),
                                      ctypes.POINTER(_c_void_p), ctypes.POINTER(_c_float), _c_void_p,
                                      _c_void_p, _c_void_p, _c_void_p, _c_size_t, _c_int, _c_int,
                                      _c_int, _c_int, _c_float, _c_void_p]),
    "cats_mlp_static": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                                 _c_int, _c_float, _c_void_p, _c_void_p]),
    "cats_mlp_static_limit": (_c_size_t, []),
    "cats_mlp_static_status": (_c_int, [ctypes.POINTER(_c_int), _c_void_p]),
    "cats_mlp_stack": (_c_int, [_c_int, ctypes.POINTER(_c_void_p), ctypes.POINTER(_c_void_p),
                                ctypes.POINTER(_c_void_p), ctypes.POINTER(_c_float), _c_void_p,
                                _c_void_p, _c_void_p, _c_void_p, _c_size_t, _c_int, _c_int,
                                _c_int, _c_int, _c_float, _c_void_p]),
    "cats_tp_exchange_bytes": (_c_size_t, [_c_int]),
    "cats_tp_exchange_alloc": (_c_int, [_c_int, ctypes.POINTER(_c_void_p), ctypes.c_char_p]),
    "cats_tp_exchange_open": (_c_int, [ctypes.c_char_p, ctypes.POINTER(_c_void_p)]),
    "cats_tp_exchange_close": (_c_int, [_c_void_p]),
    "cats_tp_exchange_free": (_c_int, [_c_void_p]),
    "cats_tp_mlp_stack": (_c_int, [_c_int, ctypes.POINTER(_c_void_p), ctypes.POINTER(_c_void_p),
                                   ctypes.POINTER(_c_void_p), ctypes.POINTER(ctypes.c_float),
                                   _c_void_p, _c_void_p, _c_void_p, _c_size_t, _c_int, _c_int,
                                   _c_int, _c_int, ctypes.c_float, _c_int, _c_int,
                                   ctypes.POINTER(_c_void_p), _c_void_p]),
    "cats_histogram": (_c_int, [_c_void_p, _c_size_t, _c_int, _c_void_p, _c_int, _c_void_p, _c_int,
                                _c_void_p]),
    "cats_histogram_threshold": (_c_int, [_c_void_p, _c_void_p, _c_int, _c_float, _c_void_p,
                                          _c_void_p]),
    "cats_uses_persistent_kernel": (_c_int, [_c_int, _c_int, _c_int, _c_int, _c_int]),
    "cats_down_dense": (_c_int, [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                 _c_void_p]),
    "cats_tail": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_float, _c_int, _c_int,
                           _c_int, _c_void_p]),
    "cats_rope_cache": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                 _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p]),
    "cats_transpose": (_c_int, [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p]),
    "cats_read_counters": (_c_int, [_c_void_p, ctypes.POINTER(_c_int), ctypes.POINTER(_c_int),
                                    _c_void_p]),
    "cats_export_list": (_c_int, [_c_void_p, _c_size_t, _c_int, _c_int, _c_int, _c_int,
                                  _c_void_p, _c_void_p, _c_void_p]),
}

_lock = threading.Lock()
_lib = None


def lib_path() -> str:
    return _build.LIB_PATH


def lib() -> ctypes.CDLL:
    """Load (building first if the sources are newer) and return the C-ABI library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(_build.LIB_PATH) or (
            not _build.is_current() and os.environ.get("CATS_B200_NO_REBUILD") != "1"
        ):
            _build.build()
        handle = ctypes.CDLL(_build.LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is missing
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, what: str = "cats") -> None:
    """Raise ``RuntimeError`` for a non-zero status code (the reference exits the process here:
    flash_gemv/csrc/cuda/fuse_gemv_cmp_cuda.cu:2397-2400)."""
    if status == 0:
        return
    L = lib()
    msg = L.cats_status_string(status).decode()
    if status == -6:
        msg += ": " + L.cats_last_cuda_error().decode()
    raise RuntimeError(f"{what}: {msg} (status {status})")
