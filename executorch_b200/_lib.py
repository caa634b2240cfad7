"""Loads the in-tree CUDA library and declares its C ABI (include/etb200_sampler.h).

There is deliberately no fallback: if the library is missing or no CUDA device is usable,
callers get an exception, never a silent CPU path.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libetb200_sampler.so")

OK = 0x00
INTERNAL = 0x01
INVALID_STATE = 0x02
NOT_SUPPORTED = 0x10
INVALID_ARGUMENT = 0x12
MEMORY_ALLOCATION_FAILED = 0x21

DTYPE_HALF, DTYPE_FLOAT, DTYPE_BFLOAT16, DTYPE_UINT16 = 5, 6, 15, 27

# every symbol include/etb200_sampler.h declares: (restype, argtypes)
class RowOptions(C.Structure):
    """etb200_row_options_t of include/etb200_sampler.h."""
    _fields_ = [("temperature_device", C.c_void_p), ("topp_device", C.c_void_p), ("topk_device", C.c_void_p),
                ("scale", C.c_float), ("edit_offsets_device", C.c_void_p), ("edit_ids_device", C.c_void_p),
                ("edit_bias_device", C.c_void_p), ("n_edits", C.c_int64)]


SYMBOLS = {
    "etb200_sampler_create": (C.c_uint32, [C.c_int32, C.c_float, C.c_float, C.c_uint64, C.c_int32,
                                           C.POINTER(C.c_void_p)]),
    "etb200_sampler_create_default": (C.c_uint32, [C.c_int32, C.c_float, C.c_int32,
                                                   C.POINTER(C.c_void_p)]),
    "etb200_sampler_destroy": (C.c_uint32, [C.c_void_p]),
    "etb200_sampler_set_temperature": (C.c_uint32, [C.c_void_p, C.c_float]),
    "etb200_sampler_set_inv_temperature": (C.c_uint32, [C.c_void_p, C.c_float]),
    "etb200_sampler_set_topk": (C.c_uint32, [C.c_void_p, C.c_int32]),
    "etb200_sampler_get_rng_state": (C.c_uint32, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "etb200_sampler_set_rng_state": (C.c_uint32, [C.c_void_p, C.c_uint64]),
    "etb200_sampler_sample": (C.c_uint32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                           C.POINTER(C.c_int32)]),
    "etb200_sampler_sample_rows": (C.c_uint32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64,
                                                C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "etb200_sampler_sample_rows_ex": (C.c_uint32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64,
                                                   C.c_void_p, C.c_void_p, C.POINTER(RowOptions), C.c_void_p]),
    "etb200_sampler_sample_rows_scatter": (C.c_uint32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64,
                                                        C.c_int64, C.c_void_p, C.POINTER(C.c_void_p),
                                                        C.c_int32, C.c_int64, C.c_void_p]),
    "etb200_sampler_sample_rows_exchange": (C.c_uint32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64,
                                                         C.c_int64, C.c_void_p, C.POINTER(C.c_void_p),
                                                         C.POINTER(C.c_void_p), C.c_int32, C.c_int32,
                                                         C.c_int64, C.c_uint64, C.c_void_p]),
    "etb200_sampler_get_status": (C.c_uint32, [C.c_void_p, C.POINTER(C.c_int32)]),
    "etb200_sampler_sample_rows_host": (C.c_uint32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64,
                                                     C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "etb200_sample_rows_static": (C.c_uint32, [C.c_int32, C.c_float, C.c_float, C.c_void_p, C.c_int32,
                                               C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "etb200_static_last_error_message": (C.c_char_p, []),
    "etb200_selftest_expf": (C.c_uint32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "etb200_sampler_set_wait_limit_ns": (C.c_uint32, [C.c_void_p, C.c_uint64]),
    "etb200_sampler_set_kernel_choice": (C.c_uint32, [C.c_void_p, C.c_int32]),
    "etb200_sampler_last_retry_count": (C.c_uint32, [C.c_void_p, C.POINTER(C.c_int32)]),
    "etb200_sampler_launch_count": (C.c_uint32, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "etb200_last_error_message": (C.c_char_p, []),
    "etb200_sampler_abi_version": (C.c_uint32, []),
}


class SamplerError(RuntimeError):
    """An error code returned by the C ABI (values of executorch::runtime::Error)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"etb200 error 0x{code:02x}: {message}")
        self.code = code


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is not built. Run `python -m executorch_b200.build` (needs nvcc); "
            "the sampler has no CPU implementation to fall back to.")
    lib = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != OK:
        raise SamplerError(code, load().etb200_last_error_message().decode())
