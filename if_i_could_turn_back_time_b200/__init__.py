"""B200-native fused 4-bit dequantise-and-multiply behind a Jenks-quantized Linear.

Public surface:
    JenksQuantLinear, quantize_module   -- drop-in for the reference's QuantLinear
    QuantSpec, PackedWeight, pack_weight -- packed formats and the host packer
    ops.linear / ops.dequantize / ops.fwht_block / ops.GroupedGemv -- kernels
All compute goes through libjq.so (include/jq.h); nothing falls back to CPU.
"""
from .spec import QuantSpec, algorithmic_bytes  # noqa: F401
from .pack import PackedWeight, pack_weight  # noqa: F401
from . import ops  # noqa: F401
from .linear import JenksQuantLinear, quantize_module  # noqa: F401
from .conv import JenksQuantConv2d  # noqa: F401

__all__ = ["QuantSpec", "PackedWeight", "pack_weight", "ops", "JenksQuantLinear", "JenksQuantConv2d", "quantize_module",
           "algorithmic_bytes"]
