"""Two-class Jenks prune mask on the GPU, O(n).

Mirrors ``Linear_Mask`` / ``Bias_Mask`` of the reference
(Python_Jenks_Test/Jenks_Tests/cuda_helpers.py:378-411): sort the flattened
scores ascending, find the natural break that minimises the two-class
within-class variance, put 1 at every element from the break upwards, and
report the goodness of variance fit.  The reference's kernel is O(n^2); this
one is a float64 prefix-sum evaluation in one pass (csrc/jenks2.cu).
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from . import _lib


def jenks2_break(sorted_vals: torch.Tensor, return_var: bool = False):
    """sorted_vals: 1-D ascending fp32 CUDA tensor -> (break index, min var, GVF[, var])."""
    lib = _lib.load()
    if not sorted_vals.is_cuda:
        raise RuntimeError("jenks2_break runs on CUDA tensors only (there is no CPU path)")
    v = sorted_vals.contiguous().float()
    n = v.numel()
    out = torch.empty(3, dtype=torch.float64, device=v.device)
    var = torch.empty(n, dtype=torch.float64, device=v.device) if return_var else None
    wsb = lib.jq_jenks2_workspace_bytes(n)
    ws = torch.empty(wsb, dtype=torch.uint8, device=v.device)
    with torch.cuda.device(v.device):
        st = lib.jq_jenks2_break(ctypes.c_void_p(v.data_ptr()), n, None if var is None else ctypes.c_void_p(var.data_ptr()),
                                 ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(ws.data_ptr()), wsb,
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(st, "jq_jenks2_break")
    o = out.cpu()
    res = (int(o[0].item()), float(o[1].item()), float(o[2].item()))
    return res + (var,) if return_var else res


def linear_mask(scores: torch.Tensor) -> Tuple[torch.Tensor, float]:
    """Mask (same shape, 1 = keep) and GVF, as the reference's Linear_Mask."""
    flat = scores.reshape(-1).float()
    sorted_vals, order = flat.sort()
    brk, _, gvf = jenks2_break(sorted_vals)
    mask = torch.zeros_like(flat)
    mask[order[brk:]] = 1
    return mask.reshape(scores.shape), gvf
