"""Packed checkpoints: the on-disk form of the packed formats.

The reference saves plain float ``state_dict``s with ``torch.save``
(Python_Jenks_Test/Jenks_Tests/training_loop.py:318-320) and loads them back
into ``nn.Sequential`` models whose Linear layers sit at keys like
``1.weight`` / ``1.bias`` (Python_Jenks_Test/Jenks_Tests/QuantNetworkTest.py:111-115).
A packed checkpoint keeps every non-Linear entry as it is and replaces each
2-D ``<prefix>.weight`` by

    <prefix>.qweight   uint8 [N, stride/2]
    <prefix>.scales    fp16  [N, K/g]        (absent when g == 0)
    <prefix>.codebook  fp16  [N, 16]         (GF4 only)
    <prefix>.meta      int32 [5] = (format id, group size, rotation block, N, K)

so it is still an ordinary ``torch.save``-able dict of tensors.
"""
from __future__ import annotations

import warnings
from typing import Dict, Iterable, Optional

import torch
import torch.nn as nn

from .linear import JenksQuantLinear
from .pack import PackedWeight, pack_weight
from .spec import QuantSpec

_FMT = {0: "e2m1", 1: "gf4"}


def pack_state_dict(state_dict: Dict[str, torch.Tensor], spec: QuantSpec,
                    only: Optional[Iterable[str]] = None, threads: int = 0) -> Dict[str, torch.Tensor]:
    """Float state_dict -> packed state_dict.  Every 2-D ``*.weight`` (or just
    the prefixes in ``only``) is quantised.  Without rotation, zeros stay
    exact zeros (E2M1 code 0; GF4 pins the zero's class to 0.0), so the mask
    the reference derives from them (Quantization_Experiments/utils.py:1507-1513)
    is implicit in the packed codes; with ``had_block`` the rotated weight has
    no zeros to keep.  A layer whose K is not a multiple of the group size or
    rotation block cannot use ``spec``: it is packed as ungrouped GF4 instead,
    with a warning, and its ``.meta`` records the format actually used."""
    only = None if only is None else set(only)
    out: Dict[str, torch.Tensor] = {}
    for key, t in state_dict.items():
        prefix = key[: -len(".weight")] if key.endswith(".weight") else None
        if prefix is not None and t.dim() == 2 and (only is None or prefix in only):
            g = spec.group_size
            fits = (not g or t.shape[1] % g == 0) and (not spec.had_block or t.shape[1] % spec.had_block == 0)
            use = spec if fits else QuantSpec("gf4", 0, 0)
            if not fits:
                warnings.warn(f"{key}: K={t.shape[1]} does not fit {spec}; packed as ungrouped GF4 instead")
            pw = pack_weight(t, use, threads=threads)
            out[prefix + ".qweight"] = pw.qweight
            if pw.scales is not None:
                out[prefix + ".scales"] = pw.scales
            if pw.codebook is not None:
                out[prefix + ".codebook"] = pw.codebook
            out[prefix + ".meta"] = torch.tensor([use.fmt_id, use.group_size, use.had_block, pw.N, pw.K], dtype=torch.int32)
        else:
            out[key] = t
    return out


def packed_weight_from(state_dict: Dict[str, torch.Tensor], prefix: str) -> PackedWeight:
    meta = [int(v) for v in state_dict[prefix + ".meta"].tolist()]
    spec = QuantSpec(_FMT[meta[0]], meta[1], meta[2])
    return PackedWeight(spec, meta[3], meta[4], state_dict[prefix + ".qweight"], state_dict.get(prefix + ".scales"),
                        state_dict.get(prefix + ".codebook"))


def linear_from_packed(pw: PackedWeight, bias: Optional[torch.Tensor] = None) -> JenksQuantLinear:
    """A committed JenksQuantLinear around already packed tensors."""
    skeleton = nn.Linear(pw.K, pw.N, bias=bias is not None)
    q = JenksQuantLinear.__new__(JenksQuantLinear)
    nn.Linear.__init__(q, pw.K, pw.N, bias=bias is not None)
    del skeleton
    q._parameters["weight"] = None
    if bias is not None:
        q.bias.requires_grad = False
        q.bias.data = bias.detach().clone().float()
    q.register_buffer("mask", None)
    q.spec = pw.spec
    q.threads = 0
    q.hard_quant = True
    q.register_buffer("qweight", pw.qweight)
    q.register_buffer("scales", pw.scales)
    q.register_buffer("codebook", pw.codebook)
    return q


def load_packed_into(model: nn.Module, state_dict: Dict[str, torch.Tensor]) -> nn.Module:
    """Replace every nn.Linear of ``model`` that has packed entries by a
    committed JenksQuantLinear, then load the remaining entries normally."""
    rest = dict(state_dict)
    for name, module in list(model.named_modules()):
        if isinstance(module, nn.Linear) and name + ".meta" in state_dict:
            pw = packed_weight_from(state_dict, name)
            new = linear_from_packed(pw, state_dict.get(name + ".bias"))
            parent = model
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            setattr(parent, parts[-1], new)
            for suffix in (".qweight", ".scales", ".codebook", ".meta", ".bias"):
                rest.pop(name + suffix, None)
    if rest:
        res = model.load_state_dict(rest, strict=False)
        # the replaced layers have no dense weight any more; anything else missing or unknown is an error
        replaced = {n + ".weight" for n, m in model.named_modules() if isinstance(m, JenksQuantLinear)}
        packed_buffers = {n + s for n, m in model.named_modules() if isinstance(m, JenksQuantLinear)
                          for s in (".qweight", ".scales", ".codebook", ".mask")}
        missing = [k for k in res.missing_keys if k not in replaced and k not in packed_buffers]
        if missing or res.unexpected_keys:
            raise RuntimeError(f"packed checkpoint does not match the model: missing {missing}, "
                               f"unexpected {list(res.unexpected_keys)}")
    return model
