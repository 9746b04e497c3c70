"""Seeded synthetic inputs for the quantized matvec: raw GGUF blocks and activations.

Every byte of a block is uniform-random, which makes the packed sub-scales, quants, codebook
indices and sign bits uniform over their bit widths; the fp16 super-scale fields are then
overwritten with finite values drawn uniformly from [lo, hi).  This is the input recipe of the
reference's own kernel test (engine/tests/test_phase30_cuda_qmatvec.py:45-57, which uses
[0.001, 0.05)); the benchmark configurations use [1e-3, 1e-2).
"""
from __future__ import annotations

import numpy as np

from .gguf_types import F16_FIELDS, TRAITS, GGUFTensorType


def synthetic_blocks(
    tensor_type: GGUFTensorType | int,
    rows: int,
    cols: int,
    rng: np.random.Generator,
    lo: float = 1e-3,
    hi: float = 1e-2,
) -> np.ndarray:
    """Raw bytes of a rows x cols tensor in `tensor_type` block layout, shape [rows, row_bytes] uint8."""
    tensor_type = GGUFTensorType(tensor_type)
    block, size = TRAITS[tensor_type]
    if cols % block:
        raise ValueError(f"cols={cols} is not a multiple of the block size {block}")
    if tensor_type is GGUFTensorType.F32:
        return rng.uniform(-1.0, 1.0, (rows, cols)).astype("<f4").view(np.uint8).reshape(rows, cols * 4)
    if tensor_type is GGUFTensorType.F16:
        return rng.uniform(-1.0, 1.0, (rows, cols)).astype("<f2").view(np.uint8).reshape(rows, cols * 2)
    nblk = cols // block
    raw = rng.integers(0, 256, (rows, nblk, size), dtype=np.uint8)
    for off in F16_FIELDS[tensor_type]:
        scale = rng.uniform(lo, hi, (rows, nblk)).astype("<f2")
        raw[:, :, off : off + 2] = scale.view(np.uint8).reshape(rows, nblk, 2)
    return raw.reshape(rows, nblk * size)


def synthetic_activations(ntok: int, cols: int, rng: np.random.Generator) -> np.ndarray:
    """fp32 N(0,1) activations, shape [ntok, cols]."""
    return rng.standard_normal((ntok, cols)).astype(np.float32)


# One decoder layer of the synthetic 27B set: (name, type, rows, cols).  A Q3_K gate/up pair, a Q4_K
# down projection and Q6_K attention projections, hidden 5120 and FFN 17408.
LAYER_SET: tuple[tuple[str, GGUFTensorType, int, int], ...] = (
    ("attn_q", GGUFTensorType.Q6_K, 6144, 5120),
    ("attn_k", GGUFTensorType.Q6_K, 1024, 5120),
    ("attn_v", GGUFTensorType.Q6_K, 1024, 5120),
    ("attn_o", GGUFTensorType.Q6_K, 5120, 6144),
    ("ffn_gate", GGUFTensorType.Q3_K, 17408, 5120),
    ("ffn_up", GGUFTensorType.Q3_K, 17408, 5120),
    ("ffn_down", GGUFTensorType.Q4_K, 5120, 17408),
)
LM_HEAD: tuple[str, GGUFTensorType, int, int] = ("output", GGUFTensorType.Q6_K, 151936, 5120)
N_LAYERS = 64

# The IQ-type sweep: (type, rows, cols).
IQ_SWEEP: tuple[tuple[GGUFTensorType, int, int], ...] = (
    (GGUFTensorType.IQ2_XXS, 17408, 5120),
    (GGUFTensorType.IQ2_S, 17408, 5120),
    (GGUFTensorType.IQ3_S, 17408, 5120),
    (GGUFTensorType.IQ4_XS, 17408, 5120),
    (GGUFTensorType.IQ4_NL, 5120, 17408),
)


def tensor_bytes(tensor_type: GGUFTensorType | int, rows: int, cols: int) -> int:
    block, size = TRAITS[GGUFTensorType(tensor_type)]
    return rows * (cols // block) * size


def layer_set_bytes() -> int:
    return sum(tensor_bytes(t, r, c) for _, t, r, c in LAYER_SET)
