"""CPU oracle for the packed 4-bit formats -- TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA path is compared against.  Only the test
suite, the smoke check and the benchmark's CPU-baseline leg may import it; the
product package never does.

Parity status: "parity unpinned".  The reference project keeps its quantized
weights as dense fp32 and has no packed 4-bit codec, no E2M1 grid, no codebook
format and no Hadamard rotation, and its repository holds no golden vectors
for this path.  What the reference does fix, and what this file follows:

* dequantize-then-linear in fp32, ``y = F.linear(x, W_hat, bias)``
  (Python_Jenks_Test/Jenks_Tests/Quantization_Experiments/layers.py:33-38);
* scale = absmax / qmax per output row, generalised here to per (row, group)
  (layers.py:23-26);
* round-to-nearest-even onto the grid (``torch.round``) and the
  "all-zero slice gets scale 1" guard
  (Quantization_Experiments/utils.py:705-710, 838-840);
* the Jenks objective: minimise the total within-class sum of squared
  deviations over contiguous splits of the ascending-sorted values, first
  minimum wins (Python_Jenks_Test/Jenks_Tests/cuda_helpers.py:151-184,
  378-395), with ``n_classes = min(k, #unique)``
  (Python_Jenks_Test/Jenks_Tests/custom_optimizer.py:118-120).

Everything is numpy; sizes are meant to finish in seconds.
"""
from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------
# E2M1 (FP4) grid: code = s e1 e0 m, bit 3 is the sign.
# --------------------------------------------------------------------------
E2M1_MAGNITUDES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_VALUES = np.concatenate([E2M1_MAGNITUDES, -E2M1_MAGNITUDES]).astype(np.float32)
# midpoints between neighbouring magnitudes, and the magnitude index a value
# exactly on the midpoint rounds to (the neighbour whose mantissa bit is 0)
_E2M1_MID = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
_E2M1_TIE = np.array([0, 2, 2, 4, 4, 6, 6], dtype=np.int64)

INV_SQRT_128 = np.float32(0.08838834764831845)


def row_stride_codes(K: int) -> int:
    """Codes per packed row: K rounded up so a row is a multiple of 16 bytes."""
    return (K + 31) // 32 * 32


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """codes uint8 [N, K] in 0..15 -> uint8 [N, stride/2]; the low nibble of
    byte j holds code 2j, the high nibble code 2j+1; padding codes are 0."""
    codes = np.asarray(codes, dtype=np.uint8)
    N, K = codes.shape
    Ks = row_stride_codes(K)
    full = np.zeros((N, Ks), dtype=np.uint8)
    full[:, :K] = codes
    return (full[:, 0::2] | (full[:, 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(qweight: np.ndarray, K: int) -> np.ndarray:
    """uint8 [N, stride/2] -> codes uint8 [N, K]."""
    q = np.asarray(qweight, dtype=np.uint8)
    N = q.shape[0]
    out = np.empty((N, q.shape[1] * 2), dtype=np.uint8)
    out[:, 0::2] = q & 0xF
    out[:, 1::2] = q >> 4
    return out[:, :K]


# --------------------------------------------------------------------------
# E2M1 quantise / dequantise
# --------------------------------------------------------------------------
def e2m1_round_codes(u: np.ndarray) -> np.ndarray:
    """Nearest E2M1 code for fp32 values u, ties to the even mantissa bit,
    saturating at +-6.  Never emits code 8 (negative zero)."""
    u = np.asarray(u, dtype=np.float32)
    a = np.abs(u)
    idx = np.zeros(a.shape, dtype=np.int64)
    for j, mid in enumerate(_E2M1_MID):
        idx = np.where(a > mid, j + 1, idx)
    for j, mid in enumerate(_E2M1_MID):
        idx = np.where(a == mid, _E2M1_TIE[j], idx)
    neg = (u < 0) & (idx != 0)
    return (idx + 8 * neg).astype(np.uint8)


def group_absmax(W: np.ndarray, g: int) -> np.ndarray:
    N, K = W.shape
    assert K % g == 0
    return np.abs(W.reshape(N, K // g, g)).max(axis=2)


def quantize_e2m1(W: np.ndarray, g: int = 32):
    """fp32 W [N,K] -> (codes uint8 [N,K], scales fp16 [N,K/g]).
    scale = fp16_rn(absmax/6), 1.0 for an all-zero group, 65504 where that overflows; u = w / fp32(scale)."""
    W = np.asarray(W, dtype=np.float32)
    N, K = W.shape
    amax = group_absmax(W, g)
    with np.errstate(over="ignore"):
        scales = (amax / np.float32(6.0)).astype(np.float16)
    # a scale that underflows to zero in fp16 would divide by zero
    scales = np.where((amax == 0) | (scales == 0), np.float16(1.0), scales).astype(np.float16)
    # one that overflows (absmax above 6 * 65504) would dequantise the whole group to inf / nan: largest finite
    # fp16 instead, the codes saturate at +-6
    scales = np.where(np.isinf(scales), np.float16(65504.0), scales).astype(np.float16)
    s32 = scales.astype(np.float32)
    u = (W.reshape(N, K // g, g) / s32[:, :, None]).astype(np.float32).reshape(N, K)
    return e2m1_round_codes(u), scales


def dequant_e2m1(codes: np.ndarray, scales: np.ndarray, g: int = 32) -> np.ndarray:
    """One fp32 multiply per weight: fp32(value(code)) * fp32(scale)."""
    N, K = codes.shape
    v = E2M1_VALUES[codes.astype(np.int64)]
    s32 = np.asarray(scales, dtype=np.float16).astype(np.float32)
    return (v.reshape(N, K // g, g) * s32[:, :, None]).astype(np.float32).reshape(N, K)


def dequant_e2m1_folded_fp16(codes: np.ndarray, scales: np.ndarray, g: int = 32) -> np.ndarray:
    """The weights the batched tensor-memory kernel multiplies by: the exact
    product value(code) * scale (13 significant bits at most) rounded once to
    fp16, because there the group scale is folded into the fp16 operand of the
    tensor-core MMA instead of being applied in fp32 after the accumulation.
    Used for the tight kernel check beside the 1e-3 gate against dequant_e2m1."""
    return dequant_e2m1(codes, scales, g).astype(np.float16).astype(np.float32)


# --------------------------------------------------------------------------
# GF4 dequantise (the quantiser lives in oracle/jenks.py)
# --------------------------------------------------------------------------
def dequant_gf4(codes: np.ndarray, codebook: np.ndarray, scales: np.ndarray | None, g: int = 0) -> np.ndarray:
    """codes [N,K], codebook fp16 [N,16], scales fp16 [N,K/g] or None."""
    N, K = codes.shape
    cb32 = np.asarray(codebook, dtype=np.float16).astype(np.float32)
    v = np.take_along_axis(cb32, codes.astype(np.int64), axis=1)
    if scales is None or g == 0:
        return v.astype(np.float32)
    s32 = np.asarray(scales, dtype=np.float16).astype(np.float32)
    return (v.reshape(N, K // g, g) * s32[:, :, None]).astype(np.float32).reshape(N, K)


# --------------------------------------------------------------------------
# Block Walsh-Hadamard rotation
# --------------------------------------------------------------------------
def fwht_block(x: np.ndarray, h: int = 128) -> np.ndarray:
    """Orthonormal Sylvester-ordered Hadamard over consecutive blocks of h
    along the last axis, in fp32: log2(h) butterfly stages with strides
    1, 2, 4, ... (a+b to the low slot, a-b to the high slot), then a single
    fp32 multiply by fp32(1/sqrt(h))."""
    x = np.asarray(x, dtype=np.float32)
    K = x.shape[-1]
    assert K % h == 0 and h & (h - 1) == 0
    y = x.reshape(-1, K // h, h).copy()
    s = 1
    while s < h:
        v = y.reshape(y.shape[0], y.shape[1], h // (2 * s), 2, s)
        a = v[:, :, :, 0, :].copy()
        b = v[:, :, :, 1, :].copy()
        v[:, :, :, 0, :] = a + b
        v[:, :, :, 1, :] = a - b
        s *= 2
    scale = np.float32(1.0 / np.sqrt(np.float64(h)))
    return (y * scale).astype(np.float32).reshape(x.shape)


def hadamard_matrix(h: int) -> np.ndarray:
    H = np.array([[1.0]])
    while H.shape[0] < h:
        H = np.block([[H, H], [H, -H]])
    return H


# --------------------------------------------------------------------------
# The operator: dequantise, rotate, fp32 linear
# --------------------------------------------------------------------------
def linear_ref(x: np.ndarray, w_hat: np.ndarray, bias: np.ndarray | None, had_block: int = 0) -> np.ndarray:
    """y = rotate(x) @ w_hat.T + bias in fp32 (float64 accumulation, rounded
    once, so the reference itself carries no summation-order noise)."""
    xt = np.asarray(x, dtype=np.float32)
    if had_block:
        xt = fwht_block(xt, had_block)
    y = xt.astype(np.float64) @ np.asarray(w_hat, dtype=np.float32).astype(np.float64).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32).astype(np.float64)
    return y.astype(np.float32)


def activation_exponent(amax: np.float32, had: bool) -> int:
    """Exponent e of the power-of-two normalisation the CUDA GEMV applies to a
    batch row: the fp32 exponent field of max|x| (before rotation) minus 127
    minus 10 with the rotation (which can grow the maximum by sqrt(128)) or
    minus 14 without, clamped to [-100, 100]; 0 for a zero or non-finite
    maximum.  x * 2^-e then stays below 2^15, inside fp16 range."""
    bits = int(np.float32(amax).view(np.uint32))
    field = (bits >> 23) & 0xFF
    if field == 0xFF or (bits & 0x7FFFFFFF) == 0:
        return 0
    return int(min(100, max(-100, field - 127 - (10 if had else 14))))


def activation_fp16_model(x: np.ndarray, had: bool) -> np.ndarray:
    """The values the CUDA GEMV multiplies the weights by: per batch row,
    x * 2^-e, rotated in fp32 (if ``had``), rounded to fp16, times 2^e.
    Scaling by a power of two commutes exactly with the fp32 butterflies, so
    this is rotate(x) rounded to 11 significant bits.  Used for the tight
    kernel check that sits beside the 1e-3 gate against unrounded fp32."""
    x = np.asarray(x, dtype=np.float32)
    out = np.empty_like(x)
    for b in range(x.shape[0]):
        amax = np.float32(np.max(np.abs(x[b]))) if x.shape[1] else np.float32(0)
        e = activation_exponent(amax, had)
        down = np.ldexp(np.float32(1.0), -e).astype(np.float32)
        up = np.ldexp(np.float32(1.0), e).astype(np.float32)
        v = x[b:b + 1] * down
        if had:
            v = fwht_block(v, 128)
        out[b] = v.astype(np.float16).astype(np.float32)[0] * up
    return out


def activation_e4m3_model(x: np.ndarray, had: bool, terms: int) -> np.ndarray:
    """The values the tensor-core kernel multiplies the weights by: per batch
    row, u = rotate(x * 2^-e) with e = exponent field of max|x| - 127 - 7
    (- 3 with rotation), so that |u| < 256; then t1 = e4m3(u), t2 = e4m3(u -
    t1), [t3 = e4m3(u - t1 - t2)], all round-to-nearest-even; the model value
    is (t1 + t2 + t3) * 2^e."""
    import torch
    x = np.asarray(x, dtype=np.float32)
    out = np.empty_like(x)
    for b in range(x.shape[0]):
        amax = np.float32(np.max(np.abs(x[b]))) if x.shape[1] else np.float32(0)
        bits = int(amax.view(np.uint32))
        field = (bits >> 23) & 0xFF
        e = 0 if (field == 0xFF or (bits & 0x7FFFFFFF) == 0) else int(min(100, max(-100, field - 127 - (3 if had else 7))))
        v = x[b:b + 1] * np.ldexp(np.float32(1.0), -e).astype(np.float32)
        if had:
            v = fwht_block(v, 128)
        r = torch.from_numpy(v[0].copy())
        tot = torch.zeros_like(r)
        for _ in range(terms):
            q = r.to(torch.float8_e4m3fn).to(torch.float32)
            tot = tot + q
            r = r - q
        out[b] = tot.numpy() * np.ldexp(np.float32(1.0), e).astype(np.float32)
    return out


def rel_err(y: np.ndarray, y_ref: np.ndarray) -> float:
    """max|y - y_ref| / max|y_ref| over the whole output."""
    y = np.asarray(y, dtype=np.float64)
    r = np.asarray(y_ref, dtype=np.float64)
    den = np.max(np.abs(r)) if r.size else 0.0
    if den == 0:
        return float(np.max(np.abs(y - r))) if r.size else 0.0
    return float(np.max(np.abs(y - r)) / den)
