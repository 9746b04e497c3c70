"""Loaders for the CPU checkers under oracle/ (test infrastructure only)."""
from __future__ import annotations

import ctypes
import importlib.util
import subprocess
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent.parent
ORACLE = REPO / "oracle"


def load_c_oracle() -> ctypes.CDLL:
    lib = ORACLE / "liboracle_qmv.so"
    src = ORACLE / "qmv_oracle.c"
    if not lib.exists() or lib.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ORACLE)], check=True, capture_output=True)
    dll = ctypes.CDLL(str(lib))
    dll.oracle_dequantize.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    dll.oracle_qmv.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                               ctypes.c_void_p, ctypes.c_void_p]
    dll.oracle_argmax_rows.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return dll


def _grid_ptr(tensor_type: int, codebooks: dict[str, bytes] | None):
    from vinf_3080ti_b200.gguf_types import CODEBOOK_OF_TYPE, GGUFTensorType

    name = CODEBOOK_OF_TYPE.get(GGUFTensorType(tensor_type))
    if name is None:
        return None, None
    buf = np.frombuffer((codebooks or {})[name], dtype=np.uint8).copy()
    return buf, buf.ctypes.data


def c_dequantize(dll, raw: np.ndarray, tensor_type: int, rows: int, cols: int, codebooks=None) -> np.ndarray:
    raw = np.ascontiguousarray(raw).reshape(-1)
    out = np.empty(rows * cols, dtype=np.float64)
    keep, grid = _grid_ptr(tensor_type, codebooks)
    rc = dll.oracle_dequantize(int(tensor_type), raw.ctypes.data, rows, cols, out.ctypes.data, grid)
    if rc:
        raise ValueError("oracle_dequantize rejected the shape")
    return out


def c_qmv(dll, raw: np.ndarray, tensor_type: int, rows: int, cols: int, x: np.ndarray, codebooks=None) -> np.ndarray:
    raw = np.ascontiguousarray(raw).reshape(-1)
    x = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
    y = np.empty((x.shape[0], rows), dtype=np.float64)
    keep, grid = _grid_ptr(tensor_type, codebooks)
    rc = dll.oracle_qmv(int(tensor_type), raw.ctypes.data, rows, cols, x.ctypes.data, x.shape[0], y.ctypes.data, grid)
    if rc:
        raise ValueError("oracle_qmv rejected the shape")
    return y


def c_argmax_rows(dll, y: np.ndarray) -> np.ndarray:
    y = np.ascontiguousarray(np.atleast_2d(y), dtype=np.float64)
    out = np.empty(y.shape[0], dtype=np.int32)
    dll.oracle_argmax_rows(y.ctypes.data, y.shape[1], y.shape[0], out.ctypes.data)
    return out


def load_reference_cpu_module():
    """The reference's own CPU runtime, if `make -C oracle ref` has built it; else None."""
    found = sorted((ORACLE / "_ref").glob("_cpu_qwen*.so"))
    if not found:
        return None
    spec = importlib.util.spec_from_file_location("_cpu_qwen", found[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_reference_cuda_module():
    """The reference's own CUDA runtime rebuilt for sm_100a, if `make -C oracle ref` has built it; else None."""
    found = ORACLE / "_ref" / "_cuda_qwen_runtime.so"
    if not found.exists():
        return None
    spec = importlib.util.spec_from_file_location("_cuda_qwen_runtime", found)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
