"""B200 (sm_100a) engine for the GGUF quantized matvec path of `vinf`: y = W x for 1..8 activation
rows with W kept in raw GGUF block layout in HBM, the fused LM-head matvec + argmax, and output-row
sharding across GPUs.  See runtime.Runtime for the drop-in interface and include/vinf_b200.h for the C ABI.
"""
from .gguf_types import CUDA_MATVEC_TYPES, GGUFTensorType, TRAITS, row_bytes  # noqa: F401

__all__ = ["CUDA_MATVEC_TYPES", "GGUFTensorType", "TRAITS", "row_bytes", "Runtime"]


def __getattr__(name):  # the runtime needs the built library; the type tables do not
    if name == "Runtime":
        from . import runtime

        return getattr(runtime, name)
    raise AttributeError(name)
