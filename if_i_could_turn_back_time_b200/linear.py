"""Drop-in quantized Linear over packed 4-bit weights.

Mirrors the operator surface of the reference's ``QuantLinear``
(Python_Jenks_Test/Jenks_Tests/Quantization_Experiments/layers.py:11-45):
constructed from an ``nn.Linear`` with the same positional arguments
``(linear_module, bitwidth=4, mask=None)``, ``forward(x)`` with ``F.linear``
broadcasting semantics, ``commit()``, attribute ``hard_quant``, buffer
``mask``; and of ``quantize_module`` (Quantization_Experiments/utils.py:1498-1524),
which swaps every ``nn.Linear`` of a model and derives the mask from the zero
weights.  What differs is what sits underneath: the weight is stored as packed
E2M1 or GF4 codes and the forward is one fused CUDA kernel instead of
``F.linear`` on a dense fp32 matrix.
"""
from __future__ import annotations

import copy
from typing import Optional

import torch
import torch.nn as nn

from . import ops
from .pack import PackedWeight, pack_weight
from .spec import QuantSpec


class JenksQuantLinear(nn.Linear):
    def __init__(self, linear_module: nn.Linear, bitwidth: int = 4, mask: Optional[torch.Tensor] = None, *,
                 fmt: str = "gf4", group_size: int = 128, had_block: int = 0, threads: int = 0):
        if bitwidth != 4:
            raise ValueError("the packed formats are 4-bit; bitwidth must be 4")
        super().__init__(linear_module.in_features, linear_module.out_features,
                         bias=(linear_module.bias is not None))
        self.weight.requires_grad = False
        self.weight.data = linear_module.weight.data.clone()
        if linear_module.bias is not None:
            self.bias.requires_grad = False
            self.bias.data = linear_module.bias.data.clone()
        self.register_buffer("mask", mask if mask is not None else torch.ones_like(self.weight.data))
        self.spec = QuantSpec(fmt, group_size, had_block)
        self.threads = threads
        self.hard_quant = False
        self.register_buffer("qweight", None)
        self.register_buffer("scales", None)
        self.register_buffer("codebook", None)

    # -- the dense weight stays readable after commit(), as the reference's
    #    scripts print and inspect module.weight (QuantNetworkTest.py:112-114)
    @property
    def weight(self):
        w = self._parameters.get("weight")
        if w is not None:
            return w
        return ops.dequantize(self.packed)

    @weight.setter
    def weight(self, value):
        nn.Module.__setattr__(self, "weight", value)

    @property
    def packed(self) -> PackedWeight:
        if self.qweight is None:
            self._pack()
        return PackedWeight(self.spec, self.out_features, self.in_features, self.qweight, self.scales, self.codebook)

    def _pack(self) -> None:
        dense = self._parameters["weight"]
        if dense is None:
            raise RuntimeError("no dense weight to pack")
        dev = dense.device
        W = (self.mask.to(dense.device) * dense.data).float()
        pw = pack_weight(W, self.spec, threads=self.threads).to(dev)
        self.qweight, self.scales, self.codebook = pw.qweight, pw.scales, pw.codebook

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.packed, self.bias)

    def weight_quantizer(self) -> torch.Tensor:
        """The dense quantised weight, the way BRECQ-style code asks for it:
        the reference's ``replace_forward.new_forward`` computes
        ``F.linear(x, module.weight_quantizer(), module.bias)``
        (Quantization_Experiments/brecq.py:321-329).  Calibration code that
        reads W_q gets the dequantised matrix; ``attach_packed_forward`` puts
        the fused kernel behind the same ``new_forward`` hook."""
        return ops.dequantize(self.packed)

    def commit(self) -> None:
        """Pack (if not done yet) and drop the dense fp32 weight."""
        with torch.no_grad():
            _ = self.packed
            self._parameters["weight"] = None
            self.hard_quant = True

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"fmt={self.spec.fmt}, group_size={self.spec.group_size}, had_block={self.spec.had_block}")


def attach_packed_forward(module: nn.Module, quantizer) -> nn.Module:
    """The packed counterpart of the reference's ``replace_forward``
    (Quantization_Experiments/brecq.py:305-331) for a Linear: ``quantizer`` is
    an AdaRound-style callable whose call returns the quantised weight W_q
    (``AdaRoundQuantizer.forward``, brecq.py:81-92, once its rounding is
    hard).  W_q is packed once, ``module.weight_quantizer`` keeps returning
    the dense W_q for code that inspects it, and ``module.forward`` becomes
    the fused kernel over the packed weight instead of ``F.linear(x, W_q,
    bias)``.  W_q must lie on a grid the format represents exactly for the two
    forwards to agree bit for bit; otherwise it is re-quantised by the packer.
    Returns the module."""
    if not isinstance(module, nn.Linear):
        raise TypeError("attach_packed_forward handles nn.Linear modules")
    with torch.no_grad():
        w_q = quantizer().detach()
    spec = getattr(module, "spec", None) or QuantSpec("gf4", 0, 0)
    pw = pack_weight(w_q.float(), spec).to(w_q.device)
    module.weight_quantizer = quantizer
    module.packed_weight = pw

    def new_forward(x, _m=module):
        return ops.linear(x, _m.packed_weight, _m.bias)

    module.forward = new_forward
    return module


def quantize_module(module, bitwidth: int = 4, **spec_kwargs):
    """Recursively replace ``nn.Linear`` layers by ``JenksQuantLinear``; the
    mask of each layer is taken from its zero weights, as in the reference's
    ``quantize_module`` (Quantization_Experiments/utils.py:1501-1513).  The
    reference multiplies by the mask after quantising (layers.py:37,43); here
    the masked weight is packed and both formats keep exact zeros: E2M1 code 0
    is 0, and a GF4 row that contains a zero pins the codebook entry of the
    zero's class to 0.0.  With ``had_block`` the packed weight is the rotated
    matrix, whose entries are not zero where the original was: the rotation
    trades the sparsity pattern for accuracy, and only the unrotated formats
    keep pruned weights at zero."""
    if isinstance(module, JenksQuantLinear):
        return module
    if isinstance(module, nn.Linear):
        mask = (module.weight.data != 0).float()
        return JenksQuantLinear(module, bitwidth, mask=mask, **spec_kwargs)
    if isinstance(module, nn.Conv2d) and module.groups == 1 and not isinstance(module.padding, str):
        from .conv import JenksQuantConv2d
        if isinstance(module, JenksQuantConv2d):
            return module
        mask = (module.weight.data != 0).float()
        return JenksQuantConv2d(module, bitwidth, mask=mask, **spec_kwargs)
    if isinstance(module, list):
        return [quantize_module(m, bitwidth, **spec_kwargs) for m in module]
    module = copy.deepcopy(module)
    for name, child in module.named_children():
        setattr(module, name, quantize_module(child, bitwidth, **spec_kwargs))
    return module
