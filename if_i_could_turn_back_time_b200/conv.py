"""Drop-in quantized Conv2d over the packed 4-bit formats.

Mirrors the reference's ``QuantConv2d`` surface
(Python_Jenks_Test/Jenks_Tests/Quantization_Experiments/layers.py:48-97):
built from an ``nn.Conv2d`` with ``(conv_module, bitwidth=4, mask=None)``,
``forward`` = ``F.conv2d(x, W_hat, bias, stride, padding, dilation, groups)``,
``commit()``.  The weight ``[O, I, kh, kw]`` is packed as the matrix
``[O, I*kh*kw]`` and the convolution runs as an implicit GEMM: ``F.unfold``
lays out the receptive fields (plumbing), the fused packed kernels do the
multiply (the tensor-core path when the batch of output positions is large
and the format is E2M1 g32).  groups must be 1.
"""
from __future__ import annotations

import warnings
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .pack import PackedWeight, pack_weight
from .spec import QuantSpec


class JenksQuantConv2d(nn.Conv2d):
    def __init__(self, conv_module: nn.Conv2d, bitwidth: int = 4, mask: Optional[torch.Tensor] = None, *,
                 fmt: str = "gf4", group_size: int = 0, had_block: int = 0, threads: int = 0):
        if bitwidth != 4:
            raise ValueError("the packed formats are 4-bit; bitwidth must be 4")
        if conv_module.groups != 1:
            raise ValueError("grouped convolutions are not supported")
        if isinstance(conv_module.padding, str):
            raise ValueError("string padding modes are not supported")
        super().__init__(conv_module.in_channels, conv_module.out_channels, conv_module.kernel_size,
                         conv_module.stride, conv_module.padding, conv_module.dilation, conv_module.groups,
                         bias=(conv_module.bias is not None))
        self.weight.requires_grad = False
        self.weight.data = conv_module.weight.data.clone()
        if conv_module.bias is not None:
            self.bias.requires_grad = False
            self.bias.data = conv_module.bias.data.clone()
        self.register_buffer("mask", mask if mask is not None else torch.ones_like(self.weight.data))
        kc = self.in_channels * self.kernel_size[0] * self.kernel_size[1]
        if group_size and kc % group_size:
            warnings.warn(f"reduction length {kc} is not a multiple of the group size {group_size}: "
                          "this layer is packed as ungrouped GF4")
            group_size, fmt = 0, "gf4"
        if had_block and kc % had_block:
            warnings.warn(f"reduction length {kc} is not a multiple of the rotation block: no rotation for this layer")
            had_block = 0
        self.spec = QuantSpec(fmt, group_size, had_block)
        self.threads = threads
        self.hard_quant = False
        self.register_buffer("qweight", None)
        self.register_buffer("scales", None)
        self.register_buffer("codebook", None)

    @property
    def packed(self) -> PackedWeight:
        if self.qweight is None:
            dense = self._parameters["weight"]
            W = (self.mask.to(dense.device) * dense.data).float().reshape(self.out_channels, -1)
            pw = pack_weight(W, self.spec, threads=self.threads).to(dense.device)   # on the GPU when the weight is there
            self.qweight, self.scales, self.codebook = pw.qweight, pw.scales, pw.codebook
        kc = self.in_channels * self.kernel_size[0] * self.kernel_size[1]
        return PackedWeight(self.spec, self.out_channels, kc, self.qweight, self.scales, self.codebook)

    def weight_quantizer(self) -> torch.Tensor:
        """Dense quantised weight [O, I, kh, kw], as the Conv2d branch of the
        reference's ``replace_forward`` asks for it
        (Quantization_Experiments/brecq.py:312-319)."""
        return self.dequantized_weight()

    def dequantized_weight(self) -> torch.Tensor:
        return ops.dequantize(self.packed).reshape(self.out_channels, self.in_channels, *self.kernel_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, _, H, W = x.shape
        kh, kw = self.kernel_size
        ho = (H + 2 * self.padding[0] - self.dilation[0] * (kh - 1) - 1) // self.stride[0] + 1
        wo = (W + 2 * self.padding[1] - self.dilation[1] * (kw - 1) - 1) // self.stride[1] + 1
        cols = F.unfold(x, self.kernel_size, self.dilation, self.padding, self.stride)   # [B, I*kh*kw, L]
        rows = cols.transpose(1, 2).reshape(B * ho * wo, -1).contiguous()
        y = ops.linear(rows, self.packed, self.bias)                                       # [B*L, O]
        return y.reshape(B, ho * wo, self.out_channels).transpose(1, 2).reshape(B, self.out_channels, ho, wo)

    def commit(self) -> None:
        with torch.no_grad():
            _ = self.packed
            self._parameters["weight"] = None
            self.hard_quant = True
