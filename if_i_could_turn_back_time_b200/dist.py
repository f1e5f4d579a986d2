"""Row-sharded execution across GPUs: one process per GPU, torch.distributed.

Output rows are independent (row n needs only its own codes, scales and
codebook plus the full activation), so a packed matrix shards by rows with no
weight movement at run time; the only exchange is an all-gather of the output
slices.  The reference has no multi-device path at all (single process,
``device = 'cuda' if ... else 'cpu'`` at
Python_Jenks_Test/Jenks_Tests/QuantNetworkTest.py:19).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .pack import PackedWeight


def shard_bounds(N: int, rank: int, world: int) -> Tuple[int, int]:
    """Rows [lo, hi) of rank ``rank``; N must divide evenly so that the
    gathered output is a plain concatenation."""
    if N % world:
        raise ValueError(f"N={N} does not divide over {world} ranks")
    per = N // world
    return rank * per, (rank + 1) * per


def shard_rows(pw: PackedWeight, rank: int, world: int) -> PackedWeight:
    lo, hi = shard_bounds(pw.N, rank, world)
    return pw.rows(lo, hi)


def gather_rows(y_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """[..., N/P] on every rank -> [..., N] on every rank (rank-major concat
    along the last dim).  One collective on the caller's current stream."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    lead = y_local.shape[:-1]
    n = y_local.shape[-1]
    flat = y_local.reshape(-1, n).contiguous()
    out = torch.empty((world, flat.shape[0], n), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out.view(-1), flat.view(-1), group=group)
    return out.permute(1, 0, 2).reshape(*lead, world * n)


class RowShardedLinear(torch.nn.Module):
    """A packed Linear whose rows live on ``world`` GPUs; forward computes the
    local slice with the fused kernel and all-gathers the slices."""

    def __init__(self, pw_full: PackedWeight, bias: Optional[torch.Tensor] = None,
                 group: Optional[dist.ProcessGroup] = None, device=None):
        super().__init__()
        self.group = group
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.lo, self.hi = shard_bounds(pw_full.N, rank, world)
        self.packed = pw_full.rows(self.lo, self.hi)
        if device is not None:
            self.packed = self.packed.to(device)
        self.bias = None if bias is None else bias[self.lo:self.hi].to(self.packed.qweight.device).float()
        self.out_features = pw_full.N
        self.in_features = pw_full.K

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from . import ops
        return gather_rows(ops.linear(x, self.packed, self.bias), self.group)
