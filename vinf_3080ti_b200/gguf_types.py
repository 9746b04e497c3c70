"""GGUF tensor type ids and block traits for the quantized matvec path.

The ids and (block elements, block bytes) pairs follow the reference's three copies of the
same table: engine/csrc/common/qwen_quant.cuh:17-58 (CUDA), engine/csrc/cpu/qwen_cpu.c:21-43 (C)
and engine/src/vinf/gguf/parser.py:33-94 (Python).
"""
from __future__ import annotations

from enum import IntEnum


class GGUFTensorType(IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2  # known to GGUF, but no matvec kernel exists for it (upload raises ValueError)
    Q8_0 = 8
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    IQ2_XXS = 16
    IQ2_XS = 17
    IQ3_XXS = 18
    IQ4_NL = 20
    IQ3_S = 21
    IQ2_S = 22
    IQ4_XS = 23


# type -> (weights per block, bytes per block)
TRAITS: dict[GGUFTensorType, tuple[int, int]] = {
    GGUFTensorType.F32: (1, 4),
    GGUFTensorType.F16: (1, 2),
    GGUFTensorType.Q8_0: (32, 34),
    GGUFTensorType.Q2_K: (256, 84),
    GGUFTensorType.Q3_K: (256, 110),
    GGUFTensorType.Q4_K: (256, 144),
    GGUFTensorType.Q5_K: (256, 176),
    GGUFTensorType.Q6_K: (256, 210),
    GGUFTensorType.IQ4_NL: (32, 18),
    GGUFTensorType.IQ3_S: (256, 110),
    GGUFTensorType.IQ4_XS: (256, 136),
    GGUFTensorType.IQ2_XXS: (256, 66),
    GGUFTensorType.IQ2_XS: (256, 74),
    GGUFTensorType.IQ2_S: (256, 82),
    GGUFTensorType.IQ3_XXS: (256, 98),
}

# The types the matvec kernels accept (engine/src/vinf/cuda/qwen_runtime.py:10-28).
CUDA_MATVEC_TYPES = frozenset(TRAITS)

# Byte offsets of the fp16 scale fields inside one block
# (engine/tests/test_phase30_cuda_qmatvec.py:19-33); synthetic inputs keep these finite.
F16_FIELDS: dict[GGUFTensorType, tuple[int, ...]] = {
    GGUFTensorType.Q8_0: (0,),
    GGUFTensorType.IQ4_NL: (0,),
    GGUFTensorType.Q4_K: (0, 2),
    GGUFTensorType.Q5_K: (0, 2),
    GGUFTensorType.Q6_K: (208,),
    GGUFTensorType.Q3_K: (108,),
    GGUFTensorType.Q2_K: (80, 82),
    GGUFTensorType.IQ2_XXS: (0,),
    GGUFTensorType.IQ2_XS: (0,),
    GGUFTensorType.IQ2_S: (0,),
    GGUFTensorType.IQ3_XXS: (0,),
    GGUFTensorType.IQ4_XS: (0,),
    GGUFTensorType.IQ3_S: (0,),
}

# Codebook a type needs at run time: name -> (bytes, entries x values per entry).
# The tables are data of the GGUF format; they are handed to the runtime by the caller
# (the reference passes IQ3_S's the same way: engine/csrc/megakernel/qwen_runtime.cu:1272-1297).
CODEBOOK_OF_TYPE: dict[GGUFTensorType, str] = {
    GGUFTensorType.IQ2_XXS: "iq2xxs_grid",
    GGUFTensorType.IQ2_XS: "iq2xs_grid",
    GGUFTensorType.IQ2_S: "iq2s_grid",
    GGUFTensorType.IQ3_XXS: "iq3xxs_grid",
    GGUFTensorType.IQ3_S: "iq3s_grid",
}
CODEBOOK_BYTES: dict[str, int] = {
    "iq2xxs_grid": 2048,
    "iq2xs_grid": 4096,
    "iq2s_grid": 8192,
    "iq3xxs_grid": 1024,
    "iq3s_grid": 2048,
}


def row_bytes(tensor_type: GGUFTensorType | int, cols: int) -> int:
    block, size = TRAITS[GGUFTensorType(tensor_type)]
    if cols <= 0 or cols % block:
        raise ValueError(f"cols={cols} must be a positive multiple of the block size {block}")
    return cols // block * size
