"""Description of a packed weight format."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class QuantSpec:
    fmt: str = "gf4"          # "gf4" | "e2m1"
    group_size: int = 128     # codes per fp16 scale; 0 = no scales (gf4 only)
    had_block: int = 0        # 0 or 128: block Hadamard rotation of the input

    def __post_init__(self):
        if self.fmt not in ("gf4", "e2m1"):
            raise ValueError(f"unknown format {self.fmt!r}")
        if self.fmt == "e2m1" and self.group_size == 0:
            raise ValueError("e2m1 needs a group size")
        if self.group_size < 0 or self.group_size % 32:
            raise ValueError("group_size must be 0 or a multiple of 32")
        if self.had_block not in (0, 128):
            raise ValueError("had_block must be 0 or 128")

    @property
    def fmt_id(self) -> int:
        return 0 if self.fmt == "e2m1" else 1


def row_stride_codes(K: int) -> int:
    return (K + 31) // 32 * 32


def algorithmic_bytes(spec: QuantSpec, N: int, K: int, B: int, x_bytes: int, y_bytes: int, bias: bool = False) -> int:
    """Bytes one call must move: codes + scales + codebook + activations in
    and out (+ bias); no padding, nothing read twice."""
    n = N * K // 2
    if spec.group_size:
        n += (N * K // spec.group_size) * 2
    if spec.fmt == "gf4":
        n += N * 32
    n += B * K * x_bytes + B * N * y_bytes
    if bias:
        n += N * 4
    return n
