"""ctypes binding of the C ABI declared in include/int4matmul_b200.h.

`load()` raises if the shared library has not been built: there is no fallback of any kind.
"""
from __future__ import annotations

import ctypes
import os

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libint4matmul_b200.so")
_lib = None

OK = 0
ERR_BITS, ERR_UNSUPPORTED, ERR_SHAPE, ERR_NULL, ERR_ALIGN = 1, 2, 3, 4, 5
ERR_WORKSPACE, ERR_LAUNCH, ERR_MASK, ERR_DEVICE, ERR_TIMEOUT, ERR_TOO_LARGE = 6, 7, 8, 9, 10, 11

PATH_AUTO, PATH_STREAM, PATH_TCGEN05, PATH_TCGEN05_SINGLE_CTA = 0, 1, 2, 3
PATH_STATIC_WEIGHTS = 0x100000      # I4MM_PATH_STATIC_WEIGHTS: or-ed into a path (see the header)

# every symbol the header declares, with its ctypes signature
_SIGNATURES = {
    "i4mm_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "i4mm_last_cuda_error": (ctypes.c_int, []),
    "i4mm_version": (ctypes.c_int, []),
    "i4mm_launch_count": (ctypes.c_ulonglong, []),
    "i4mm_last_launch_shape": (ctypes.c_int, []),
    "i4mm_workspace_bytes": (ctypes.c_size_t, []),
    "i4mm_quant_matmul": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                         ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                         ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "i4mm_quant_matmul_gather": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                                ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                                ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "i4mm_ipc_handle_bytes": (ctypes.c_size_t, []),
    "i4mm_peer_buffer_create": (ctypes.c_int, [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]),
    "i4mm_peer_buffer_open": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]),
    "i4mm_peer_buffer_close": (ctypes.c_int, [ctypes.c_void_p]),
    "i4mm_peer_buffer_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "i4mm_gather_flags_bytes": (ctypes.c_size_t, [ctypes.c_int64]),
    "i4mm_gather_sync": (ctypes.c_int, [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                        ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]),
    "i4mm_quant_matvec_static": (ctypes.c_int, [ctypes.c_int, ctypes.c_int,
                                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                                ctypes.c_void_p]),
    "i4mm_device_status": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "i4mm_static_device_status": (ctypes.c_int, [ctypes.c_void_p]),
    "i4mm_row_norm": (ctypes.c_int, [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                     ctypes.c_void_p]),
    "i4mm_sparse_pack": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]),
    "i4mm_check_mask": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]),
}


def library_path() -> str:
    return _LIB_PATH


def exported_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def load() -> ctypes.CDLL:
    """Load libint4matmul_b200.so and attach signatures.  Raises OSError if it was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise OSError(f"{_LIB_PATH} is missing: build it with `python -m int4matmul_kernels_b200._build`; "
                          "there is no CPU or PyTorch fallback")
        lib = ctypes.CDLL(_LIB_PATH)
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def status_string(status: int) -> str:
    return load().i4mm_status_string(int(status)).decode()
