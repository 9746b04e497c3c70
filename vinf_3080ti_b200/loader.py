"""Weights of a parsed GGUF file into HBM, every tensor resident.

The reference decides per tensor whether it fits the 12 GB card (engine/src/vinf/gguf/residency.py:256-354), mmaps the
file and uploads tensor after tensor with a blocking copy (engine/src/vinf/cuda/qwen_runtime.py:68-86 over
GGUFFile.mmap_tensor, engine/src/vinf/gguf/parser.py:153-159).  With 180 GB of HBM there is nothing to plan: every
matrix the matvec path can run goes to the device, read from the file by several threads into pinned staging while
earlier chunks are already on their way over PCIe (Runtime.upload_file).

`gguf` is any object with the reference's parsed-file interface: `.path`, and `.tensors[name]` records with
`.tensor_type`, `.dimensions` (fastest first), `.absolute_offset` and `.nbytes`.  The GGUF parser itself is not part
of this library.
"""
from __future__ import annotations

from typing import Iterable

from .gguf_types import CUDA_MATVEC_TYPES


def matvec_shape(tensor) -> tuple[int, int]:
    """(cols, rows) of a GGUF tensor record: dimension 0 is the fastest one (engine/src/vinf/cuda/qwen_runtime.py:75-78)."""
    cols = int(tensor.dimensions[0])
    rows = 1
    for dim in tensor.dimensions[1:]:
        rows *= int(dim)
    return cols, rows


def is_matrix(tensor) -> bool:
    """A tensor the matvec path runs: two or more dimensions and a type it has a kernel for.  (One-dimensional F32
    tensors - norm weights, biases - belong to the element-wise ops, which are not part of this library.)"""
    return len(tensor.dimensions) >= 2 and int(tensor.tensor_type) in {int(t) for t in CUDA_MATVEC_TYPES}


def upload_gguf_tensor(rt, gguf, name: str, *, device_name: str | None = None, threads: int = 4) -> int:
    """One tensor; returns its bytes.  ValueError for a type without a kernel, like the reference's wrapper."""
    tensor = gguf.tensors[name]
    if int(tensor.tensor_type) not in {int(t) for t in CUDA_MATVEC_TYPES}:
        raise ValueError(f"{name}: no CUDA matvec for {getattr(tensor.tensor_type, 'name', tensor.tensor_type)}")
    cols, rows = matvec_shape(tensor)
    rt.upload_file(device_name or name, gguf.path, int(tensor.absolute_offset), int(tensor.nbytes), int(tensor.tensor_type), cols, rows, threads)
    return int(tensor.nbytes)


def load_matrices(rt, gguf, names: Iterable[str] | None = None, *, threads: int = 8) -> dict[str, int]:
    """Every matrix of the file (or the named ones) into HBM; returns {name: bytes}.  Tensors are taken in file order, so
    the readers walk the file front to back."""
    chosen = list(names) if names is not None else [n for n, t in gguf.tensors.items() if is_matrix(t)]
    chosen.sort(key=lambda n: int(gguf.tensors[n].absolute_offset))
    return {name: upload_gguf_tensor(rt, gguf, name, threads=threads) for name in chosen}
