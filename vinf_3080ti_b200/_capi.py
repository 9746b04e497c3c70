"""ctypes binding of libvinf_b200.so (the C ABI declared in include/vinf_b200.h).

The library is the only compute path: loading fails loudly when it has not been built, there is no
CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_int, c_size_t, c_uint64, c_void_p
from pathlib import Path

# VINF_B200_LIB points at another build of the same library (a debug or experimental build)
LIB_PATH = Path(os.environ.get("VINF_B200_LIB") or Path(__file__).resolve().parent / "libvinf_b200.so")

OK, ERR_KEY, ERR_VALUE, ERR_TYPE, ERR_MEMORY, ERR_CUDA = range(6)


class ExtensionMissingError(RuntimeError):
    """libvinf_b200.so is not built (python -m vinf_3080ti_b200.build)."""


class TensorInfo(ctypes.Structure):
    _fields_ = [("addr", c_uint64), ("type", ctypes.c_int32), ("rows", ctypes.c_int32), ("cols", ctypes.c_int32),
                ("row_bytes", ctypes.c_int64), ("nbytes", ctypes.c_int64), ("resident", ctypes.c_int32)]


# name -> argument types (every function returns int unless listed in _RESTYPES)
SIGNATURES: dict[str, list] = {
    "vqm_last_error": [],
    "vqm_runtime_create": [c_void_p, c_size_t, POINTER(c_void_p)],
    "vqm_runtime_destroy": [c_void_p],
    "vqm_set_codebook": [c_void_p, c_char_p, c_void_p, c_size_t],
    "vqm_upload": [c_void_p, c_char_p, c_void_p, c_size_t, c_int, c_int, c_int],
    "vqm_upload_file": [c_void_p, c_char_p, c_char_p, c_uint64, c_uint64, c_int, c_int, c_int, c_int],
    "vqm_free": [c_void_p, c_char_p],
    "vqm_has": [c_void_p, c_char_p, POINTER(c_int)],
    "vqm_device_bytes": [c_void_p, POINTER(c_size_t)],
    "vqm_tensor_info": [c_void_p, c_char_p, POINTER(TensorInfo)],
    "vqm_alloc": [c_void_p, c_char_p, c_size_t, c_int],
    "vqm_bind": [c_void_p, c_char_p, c_void_p, c_size_t, c_int],
    "vqm_bind_tensor": [c_void_p, c_char_p, c_void_p, c_int, c_int, c_int],
    "vqm_release": [c_void_p, c_char_p],
    "vqm_write": [c_void_p, c_char_p, c_void_p, c_size_t, c_size_t],
    "vqm_read": [c_void_p, c_char_p, c_void_p, c_size_t, c_size_t],
    "vqm_copy": [c_void_p, c_char_p, c_size_t, c_char_p, c_size_t, c_size_t],
    "vqm_zero": [c_void_p, c_char_p],
    "vqm_zero_range": [c_void_p, c_char_p, c_size_t, c_size_t],
    "vqm_buffer_ptr": [c_void_p, c_char_p, POINTER(c_uint64), POINTER(c_size_t)],
    "vqm_buffer_elem": [c_void_p, c_char_p, POINTER(c_int)],
    "vqm_buffer_len": [c_void_p, c_char_p, POINTER(c_size_t)],
    "vqm_buffer_bytes": [c_void_p, POINTER(c_size_t)],
    "vqm_qmv": [c_void_p, c_char_p, c_char_p, c_char_p, c_int],
    "vqm_matvec": [c_void_p, c_char_p, c_void_p, c_size_t, c_void_p, c_size_t],
    "vqm_argmax": [c_void_p, c_char_p, c_int, POINTER(c_int)],
    "vqm_argmax_rows": [c_void_p, c_char_p, c_int, c_int, POINTER(c_int)],
    "vqm_qmv_argmax": [c_void_p, c_char_p, c_char_p, c_char_p, c_int, POINTER(c_int)],
    "vqm_qmv_fused": [c_void_p, c_char_p, c_char_p, c_char_p, c_int, c_int, c_char_p, c_char_p, ctypes.c_float, POINTER(c_int)],
    "vqm_argmax_result": [c_void_p, POINTER(c_uint64), POINTER(c_uint64)],
    "vqm_argmax_fetch": [c_void_p, c_int, POINTER(c_int), POINTER(ctypes.c_float)],
    "vqm_set_argmax_row_base": [c_void_p, c_char_p, c_int],
    "vqm_dequantize": [c_void_p, c_char_p, c_char_p],
    "vqm_set_gemm_min_rows": [c_void_p, c_int],
    "vqm_synchronize": [c_void_p],
    "vqm_mem_info": [POINTER(c_size_t), POINTER(c_size_t)],
    "vqm_stream": [c_void_p],
    "vqm_set_stream": [c_void_p, c_void_p],
    "vqm_capture_begin": [c_void_p],
    "vqm_capture_end": [c_void_p, POINTER(c_int)],
    "vqm_graph_launch": [c_void_p, c_int],
    "vqm_graph_destroy": [c_void_p, c_int],
    "vqm_launch_count": [c_void_p, POINTER(c_uint64)],
    "vqm_exchange_create": [c_void_p, c_size_t, c_void_p, POINTER(c_uint64)],
    "vqm_exchange_open": [c_void_p, c_void_p, POINTER(c_uint64)],
    "vqm_exchange_config": [c_void_p, c_int, c_int, POINTER(c_uint64), c_size_t, c_size_t, c_int],
    "vqm_qmv_push": [c_void_p, c_char_p, c_char_p, c_char_p, c_int, c_int, c_size_t, c_int, c_int, c_int, c_int],
    "vqm_set_column_split": [c_void_p, c_int],
    "vqm_qmv_group": [c_void_p, c_int, POINTER(c_char_p), c_char_p, POINTER(c_char_p), c_int],
    "vqm_qmv_push_group": [c_void_p, c_int, POINTER(c_char_p), c_char_p, POINTER(c_char_p), c_int, c_int, POINTER(c_size_t),
                           POINTER(c_int), POINTER(c_int), c_int],
    "vqm_probe_issue_rates": [c_int, POINTER(ctypes.c_double), c_int],
    "vqm_qmv_raw": [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p],
    "vqm_qmv_argmax_static": [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
}
_RESTYPES = {"vqm_last_error": c_char_p, "vqm_runtime_destroy": None, "vqm_stream": c_void_p}

_lib: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """Loads the library once and types every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ExtensionMissingError(
            f"{LIB_PATH} is not built; run `python -m vinf_3080ti_b200.build` (needs nvcc, no GPU needed to build)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, c_int)
    _lib = lib
    return lib


_EXC = {ERR_KEY: KeyError, ERR_VALUE: ValueError, ERR_TYPE: TypeError, ERR_MEMORY: MemoryError, ERR_CUDA: RuntimeError}


def check(status: int) -> None:
    """Turns a vqm_status into the exception the reference raises for the same failure."""
    if status != OK:
        message = load().vqm_last_error().decode("utf-8", "replace")
        raise _EXC.get(status, RuntimeError)(message)
