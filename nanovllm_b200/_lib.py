"""ctypes binding of libb200attn.so, the C ABI declared in include/b200_attn.h.

No torch types cross this boundary: only raw device pointers, sizes and strides.  There is no
fallback of any kind: if the library cannot be loaded the import of the product path fails.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int32, c_int64, c_void_p

from .build import LIB_PATH, build

_lib = None

# name -> (restype, argtypes); mirrors include/b200_attn.h one to one
SIGNATURES = {
    "b200_version": (c_int32, []),
    "b200_last_error": (c_char_p, []),
    "b200_store_kvcache": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                     c_int32, c_int32, c_int32, c_int64, c_void_p]),
    "b200_decode_workspace_bytes": (c_int64, [c_int32, c_int32, c_int32, c_int32]),
    "b200_decode_attn": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_int64,
                                   c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32, c_int32,
                                   c_int32, c_float, c_void_p]),
    "b200_decode_static_scratch_bytes": (c_int64, []),
    "b200_decode_attn_static": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_int64,
                                          c_int32, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_float,
                                          c_void_p]),
    "b200_prefill_attn": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p,
                                    c_void_p, c_int64, c_int32, c_void_p, c_int64, c_int32, c_void_p, c_void_p,
                                    c_int32, c_int32, c_int32, c_int32, c_void_p, c_int32, c_int32, c_int32,
                                    c_float, c_int32, c_void_p]),
    "b200_qk_norm_rope_store": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_float,
                                          c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32,
                                          c_int32, c_int32, c_void_p]),
    "b200_unpack_decode_metadata": (c_int32, [c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p]),
    "b200_small_allreduce_buffer_bytes": (c_int64, []),
    "b200_small_allreduce_state_bytes": (c_int64, []),
    "b200_small_allreduce_max_bytes": (c_int64, []),
    "b200_small_allreduce": (c_int32, [c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_int64, c_double, c_void_p]),
    "b200_small_allreduce_status": (c_int32, [c_void_p]),
    "b200_ipc_export": (c_int32, [c_void_p, c_void_p, c_void_p]),
    "b200_ipc_open": (c_int32, [c_void_p, c_int64, c_void_p]),
    "b200_launch_count": (c_int64, []),
    "b200_device_status": (c_int32, []),
    "b200_test_inject_timeout": (c_int32, []),
}


def load():
    """Loads (building first if the library is missing or older than its sources) and returns the
    ctypes library.  B200_ATTN_REBUILD=1 forces the build."""
    global _lib
    if _lib is not None:
        return _lib
    path = build(force=bool(os.environ.get("B200_ATTN_REBUILD")))
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = the library does not match the header
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class B200AttnError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"libb200attn status {code}: {message}")
        self.code = code


def check(code: int):
    if code != 0:
        raise B200AttnError(code, load().b200_last_error().decode(errors="replace"))
