"""The reference's forward form on CPU for the packed formats -- TEST AND
BASELINE INFRASTRUCTURE ONLY (imported by tests/ and by bench.py's CPU legs).

Two paths, both straight restatements of
Python_Jenks_Test/Jenks_Tests/Quantization_Experiments/layers.py in PyTorch
on the host cores:

* ``per_call``  -- layers.py:36-38: materialise the dense fp32 weight on every
  call (there ``mask * s * (Q + Theta)``, here nibble unpack -> table lookup
  -> times the group scale), then ``F.linear`` in fp32;
* ``committed`` -- layers.py:34-35: ``F.linear`` on a weight dequantized once.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

E2M1 = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float32)
_H128 = None


def hadamard128() -> torch.Tensor:
    global _H128
    if _H128 is None:
        H = torch.ones(1, 1)
        while H.shape[0] < 128:
            H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
        _H128 = H / (128 ** 0.5)
    return _H128


def dequantize(qweight, scales, codebook, N, K, g):
    """uint8 [N, stride/2] (+ fp16 scales, fp16 codebook) -> dense fp32 [N,K]."""
    q = qweight.to(torch.int64)
    codes = torch.stack([q & 0xF, q >> 4], dim=2).reshape(N, -1)[:, :K]
    if codebook is None:
        v = E2M1[codes]
    else:
        v = torch.gather(codebook.float(), 1, codes)
    if scales is not None and g:
        v = (v.view(N, K // g, g) * scales.float().unsqueeze(2)).view(N, K)
    return v


def rotate(x, had_block):
    if not had_block:
        return x.float()
    B, K = x.shape
    return (x.float().view(B, K // 128, 128) @ hadamard128()).view(B, K)


def per_call(x, qweight, scales, codebook, bias, N, K, g, had_block):
    w = dequantize(qweight, scales, codebook, N, K, g)
    return F.linear(rotate(x, had_block), w, bias)


def committed(x, w_hat, bias, had_block):
    return F.linear(rotate(x, had_block), w_hat, bias)
