"""Host-side packers: fp32 weight matrix -> packed 4-bit tensors.

These take the place of the grid construction in the reference's
``QuantLinear.__init__`` (Python_Jenks_Test/Jenks_Tests/Quantization_Experiments/
layers.py:22-26: per-row scale, integer grid) for the packed formats.  The
arithmetic runs in the native library (multi-threaded C++); this module only
marshals tensors.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _lib
from .spec import QuantSpec, row_stride_codes


@dataclass
class PackedWeight:
    """A packed [N, K] weight matrix (tensors may live on any device)."""
    spec: QuantSpec
    N: int
    K: int
    qweight: torch.Tensor                 # uint8 [N, stride/2]
    scales: Optional[torch.Tensor]        # fp16 [N, K/g] or None
    codebook: Optional[torch.Tensor]      # fp16 [N, 16] (gf4) or None

    def to(self, device) -> "PackedWeight":
        mv = lambda t: None if t is None else t.to(device).contiguous()
        return PackedWeight(self.spec, self.N, self.K, mv(self.qweight), mv(self.scales), mv(self.codebook))

    def rows(self, lo: int, hi: int) -> "PackedWeight":
        """Row shard [lo, hi): everything in the format is per row."""
        sl = lambda t: None if t is None else t[lo:hi].contiguous()
        return PackedWeight(self.spec, hi - lo, self.K, sl(self.qweight), sl(self.scales), sl(self.codebook))

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.qweight, self.scales, self.codebook) if t is not None)


def _gpu_packable(W: torch.Tensor, spec: QuantSpec) -> bool:
    pg = spec.group_size // 32
    return W.shape[1] % 32 == 0 and 1 <= pg <= 32 and pg & (pg - 1) == 0 and W.shape[1] % spec.group_size == 0


def _pack_e2m1_cuda(W: torch.Tensor, spec: QuantSpec, rotate: bool) -> PackedWeight:
    """E2M1 quantisation on the GPU (bit-identical to the host packer); the
    weight-side rotation uses the same fp32 butterfly kernel as the operator."""
    import ctypes
    lib = _lib.load()
    from . import ops
    Wf = W.detach().float().contiguous()
    N, K = Wf.shape
    if spec.had_block and rotate:
        if K % spec.had_block:
            raise ValueError(f"K={K} is not a multiple of the rotation block {spec.had_block}")
        Wf = ops.fwht_block(Wf, spec.had_block)
    q = torch.empty((N, K // 2), dtype=torch.uint8, device=W.device)
    s = torch.empty((N, K // spec.group_size), dtype=torch.float16, device=W.device)
    with torch.cuda.device(W.device):
        st = lib.jq_pack_e2m1(ctypes.c_void_p(Wf.data_ptr()), N, K, spec.group_size, ctypes.c_void_p(q.data_ptr()),
                              ctypes.c_void_p(s.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(st, "jq_pack_e2m1")
    return PackedWeight(spec, N, K, q, s, None)


def _pack_gf4_cuda(W: torch.Tensor, spec: QuantSpec, rotate: bool) -> PackedWeight:
    """GF4 quantisation on the GPU: one CTA per row runs the same exact
    16-class Jenks dynamic programme as the host packer, bit for bit."""
    import ctypes
    lib = _lib.load()
    from . import ops
    Wf = W.detach().float().contiguous()
    N, K = Wf.shape
    g = spec.group_size
    if g and K % g:
        raise ValueError(f"K={K} is not a multiple of the group size {g}")
    if spec.had_block and rotate:
        if K % spec.had_block:
            raise ValueError(f"K={K} is not a multiple of the rotation block {spec.had_block}")
        Wf = ops.fwht_block(Wf, spec.had_block)
    q = torch.zeros((N, row_stride_codes(K) // 2), dtype=torch.uint8, device=W.device)
    s = torch.empty((N, K // g), dtype=torch.float16, device=W.device) if g else None
    cb = torch.empty((N, 16), dtype=torch.float16, device=W.device)
    P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    with torch.cuda.device(W.device):
        wsb = lib.jq_pack_gf4_workspace_bytes(K)
        ws = torch.empty(wsb, dtype=torch.uint8, device=W.device)
        st = lib.jq_pack_gf4(P(Wf), N, K, g, P(q), P(s), P(cb), P(ws), wsb,
                             ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(st, "jq_pack_gf4")
    return PackedWeight(spec, N, K, q, s, cb)


def pack_weight(W: torch.Tensor, spec: QuantSpec, threads: int = 0, rotate: bool = True) -> PackedWeight:
    """Quantise and pack W [N, K].  With ``spec.had_block`` the weight is first
    multiplied on the right by the block Hadamard matrix (fp32), so that
    ``W x == (W H)(H x)`` once the operator rotates x."""
    lib = _lib.load()
    if W.is_cuda and spec.fmt == "e2m1" and _gpu_packable(W, spec):
        return _pack_e2m1_cuda(W, spec, rotate)
    if W.is_cuda and spec.fmt == "gf4" and W.shape[1] <= 51200:
        return _pack_gf4_cuda(W, spec, rotate)
    Wf = W.detach().to("cpu", torch.float32).contiguous().clone()
    N, K = Wf.shape
    g = spec.group_size
    if g and K % g:
        raise ValueError(f"K={K} is not a multiple of the group size {g}")
    if spec.had_block and K % spec.had_block:
        raise ValueError(f"K={K} is not a multiple of the rotation block {spec.had_block}")
    wn = Wf.numpy()
    if spec.had_block and rotate:
        _lib.check(lib.jq_rotate_weights_host(wn.ctypes.data, N, K, spec.had_block, threads), "jq_rotate_weights_host")
    q = np.zeros((N, row_stride_codes(K) // 2), dtype=np.uint8)
    s = np.zeros((N, K // g), dtype=np.uint16) if g else None
    if spec.fmt == "e2m1":
        _lib.check(lib.jq_pack_e2m1_host(wn.ctypes.data, N, K, g, q.ctypes.data, s.ctypes.data, threads),
                   "jq_pack_e2m1_host")
        cb = None
    else:
        cb = np.zeros((N, 16), dtype=np.uint16)
        _lib.check(lib.jq_pack_gf4_host(wn.ctypes.data, N, K, g, q.ctypes.data,
                                        s.ctypes.data if s is not None else None, cb.ctypes.data, threads),
                   "jq_pack_gf4_host")
    as_half = lambda a: None if a is None else torch.from_numpy(a.view(np.float16).copy())
    return PackedWeight(spec, N, K, torch.from_numpy(q), as_half(s), as_half(cb))
