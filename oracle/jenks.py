"""GF4 quantiser of the CPU oracle -- TEST INFRASTRUCTURE ONLY.

k-class Jenks natural breaks per output row (k = 16), generalising the
two-class objective of Python_Jenks_Test/Jenks_Tests/cuda_helpers.py:151-184
(sorted ascending, first minimum, lower class = indices below the break;
host wrapper :378-395) with ``n_classes = min(k, #unique)`` as in
Python_Jenks_Test/Jenks_Tests/custom_optimizer.py:118-120.  The dynamic
programme itself is the C file next to this one (oracle/jenks_dp.c), loaded
through ctypes.  Parity unpinned: the reference has no k>2 implementation and
no golden vectors for it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build() -> str:
    """Compile oracle/jenks_dp.c with the Makefile beside it."""
    so = os.path.join(_HERE, "libjq_oracle.so")
    src = os.path.join(_HERE, "jenks_dp.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libjq_oracle.so"])
    return so


def _lib():
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(build())
        for name in ("jq_oracle_jenks_breaks", "jq_oracle_jenks_brute"):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        _LIB = lib
    return _LIB


def jenks_breaks(values: np.ndarray, k: int = 16, brute: bool = False):
    """values: 1-D array (any order).  Returns (uniq float64 ascending,
    counts, breaks int32[k_eff+1]) with class c = uniq[breaks[c]:breaks[c+1]]."""
    v = np.asarray(values, dtype=np.float32).astype(np.float64)
    uniq, cnt = np.unique(v, return_counts=True)
    uniq = np.ascontiguousarray(uniq + 0.0)  # -0.0 and +0.0 are one value, written +0.0
    cntd = np.ascontiguousarray(cnt.astype(np.float64))
    m = uniq.shape[0]
    ke = min(k, m)
    breaks = np.zeros(ke + 1, dtype=np.int32)
    fn = _lib().jq_oracle_jenks_brute if brute else _lib().jq_oracle_jenks_breaks
    r = fn(uniq.ctypes.data, cntd.ctypes.data, m, k, breaks.ctypes.data)
    if r != ke:
        raise RuntimeError(f"oracle jenks failed ({r})")
    return uniq, cnt, breaks


def jenks_codebook_row(u: np.ndarray, k: int = 16):
    """One row of normalised values -> (codes uint8 [K], codebook fp16 [k]).

    codebook[c] = fp16_rn(float64 mean of class c), except that when the row
    contains an exact zero the class holding it gets the entry 0.0 (pruned
    weights must dequantise to exactly zero, as the reference's
    ``mask * s * (Q + Theta)`` guarantees:
    Python_Jenks_Test/Jenks_Tests/Quantization_Experiments/layers.py:37,43);
    the partition itself is the unconstrained optimum.  Entries past the
    classes in use repeat the last entry; code = class index of the value."""
    u = np.asarray(u, dtype=np.float32)
    uniq, cnt, breaks = jenks_breaks(u, k)
    ke = breaks.shape[0] - 1
    cw = cnt.astype(np.float64) * uniq
    P1 = np.concatenate([[0.0], np.cumsum(cw)])  # sequential float64, as in the C file
    C = np.concatenate([[0.0], np.cumsum(cnt.astype(np.float64))])
    means = (P1[breaks[1:]] - P1[breaks[:-1]]) / (C[breaks[1:]] - C[breaks[:-1]])
    cb = np.empty(k, dtype=np.float16)
    cb[:ke] = means.astype(np.float16)
    cls_of_uniq = np.repeat(np.arange(ke, dtype=np.uint8), np.diff(breaks))
    z = np.searchsorted(uniq, 0.0)
    if z < uniq.shape[0] and uniq[z] == 0.0:
        cb[cls_of_uniq[z]] = np.float16(0.0)      # the zero class is pinned to 0 (order is kept: its neighbours' means
    cb[ke:] = cb[ke - 1]                           # lie strictly outside the class's own range, which contains 0)
    pos = np.searchsorted(uniq, u.astype(np.float64))
    return cls_of_uniq[pos], cb


def quantize_gf4(W: np.ndarray, g: int = 0, k: int = 16):
    """fp32 W [N,K] -> (codes uint8 [N,K], codebook fp16 [N,k], scales fp16
    [N,K/g] or None).  With groups, scale = fp16_rn(group absmax) (1.0 for an
    all-zero group or one whose absmax underflows fp16) and Jenks runs on
    u = w / fp32(scale); without groups (g == 0) Jenks runs on the raw row."""
    W = np.asarray(W, dtype=np.float32)
    N, K = W.shape
    if g:
        assert K % g == 0
        amax = np.abs(W.reshape(N, K // g, g)).max(axis=2)
        scales = amax.astype(np.float16)
        scales = np.where((amax == 0) | (scales == 0) | ~np.isfinite(scales), np.float16(1.0), scales).astype(np.float16)
        U = (W.reshape(N, K // g, g) / scales.astype(np.float32)[:, :, None]).astype(np.float32).reshape(N, K)
    else:
        scales = None
        U = W
    codes = np.empty((N, K), dtype=np.uint8)
    cb = np.empty((N, k), dtype=np.float16)
    for n in range(N):
        codes[n], cb[n] = jenks_codebook_row(U[n], k)
    return codes, cb, scales


def two_class_break_reference_form(sorted_vals: np.ndarray) -> int:
    """The reference's two-class search restated in float64: var[i] =
    SSD(v[:i]) + SSD(v[i:]) with the class means, break = first argmin
    (cuda_helpers.py:151-184, argmin at :387)."""
    v = np.asarray(sorted_vals, dtype=np.float64)
    n = v.shape[0]
    var = np.empty(n)
    for i in range(n):
        a, b = v[:i], v[i:]
        var[i] = (((a - a.mean()) ** 2).sum() if i else 0.0) + ((b - b.mean()) ** 2).sum()
    return int(np.argmin(var))
