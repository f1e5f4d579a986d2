"""The product's host packer (C++, divide-and-conquer Jenks) against the
oracle (plain O(k m^2) DP, numpy): bit-exact codes, scales and codebooks."""
import hashlib
import os

import numpy as np
import pytest
import torch

import if_i_could_turn_back_time_b200 as jq
from oracle import formats, jenks


def _same(pw, codes, scales, cb):
    assert np.array_equal(pw.qweight.numpy(), formats.pack_nibbles(codes))
    if scales is not None:
        assert np.array_equal(pw.scales.numpy().view(np.uint16), scales.view(np.uint16))
    else:
        assert pw.scales is None
    if cb is not None:
        assert np.array_equal(pw.codebook.numpy().view(np.uint16), cb.view(np.uint16))


@pytest.mark.parametrize("N,K,g", [(8, 64, 32), (5, 4096, 32), (16, 1024, 64), (3, 256, 128)])
def test_e2m1_packer_bit_exact(N, K, g):
    rng = np.random.default_rng(N * K)
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    W[0, :g] = 0  # an all-zero group
    W[rng.random(W.shape) < 0.01] *= 10
    pw = jq.pack_weight(torch.from_numpy(W), jq.QuantSpec("e2m1", g, 0))
    _same(pw, *formats.quantize_e2m1(W, g), None)


def test_e2m1_ties_and_saturation():
    # values exactly on the rounding midpoints, group absmax 6 -> scale 1
    row = np.array([6, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -5.0, -6] + [0] * 20, dtype=np.float32)
    W = np.stack([row, row * 0.5])
    pw = jq.pack_weight(torch.from_numpy(W), jq.QuantSpec("e2m1", 32, 0))
    _same(pw, *formats.quantize_e2m1(W, 32), None)


def test_e2m1_scale_beyond_fp16_is_clamped():
    """absmax / 6 above the fp16 range: the scale is the largest finite fp16, the codes saturate, nothing becomes inf."""
    W = np.zeros((2, 64), dtype=np.float32)
    W[0, :32] = np.linspace(-5e5, 5e5, 32)          # absmax / 6 = 83333 > 65504
    W[0, 32:] = np.linspace(-3.9e5, 3.9e5, 32)      # absmax / 6 = 65000 < 65504: untouched
    W[1, :32] = 3.0e38
    pw = jq.pack_weight(torch.from_numpy(W), jq.QuantSpec("e2m1", 32, 0))
    codes, scales = formats.quantize_e2m1(W, 32)
    _same(pw, codes, scales, None)
    assert scales[0, 0] == np.float16(65504) and scales[1, 0] == np.float16(65504) and np.isfinite(scales).all()
    assert np.isfinite(formats.dequant_e2m1(codes, scales, 32)).all()


@pytest.mark.parametrize("N,K,g", [(12, 1024, 128), (6, 2048, 128), (4, 4096, 128), (9, 512, 64), (7, 300, 0),
                                    (10, 100, 0), (3, 784, 0)])
def test_gf4_packer_bit_exact(N, K, g):
    rng = np.random.default_rng(N + K)
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    W[rng.random(W.shape) < 0.001] *= 10
    pw = jq.pack_weight(torch.from_numpy(W), jq.QuantSpec("gf4", g, 0))
    c, cb, s = jenks.quantize_gf4(W, g)
    _same(pw, c, s, cb)
    assert np.all(np.diff(cb.astype(np.float32), axis=1) >= 0)  # codebooks ascend


def test_gf4_packer_ties_duplicates_and_sparse_rows():
    rng = np.random.default_rng(11)
    cases = [rng.integers(-5, 6, size=(16, 256)).astype(np.float32),
             np.round(rng.standard_normal((16, 512)) * 8).astype(np.float32) / 8,
             np.zeros((3, 64), dtype=np.float32)]
    sparse = (rng.standard_normal((10, 300)) * 0.1).astype(np.float32)
    sparse[rng.random(sparse.shape) < 0.95] = 0
    cases.append(sparse)
    for W in cases:
        pw = jq.pack_weight(torch.from_numpy(W), jq.QuantSpec("gf4", 0, 0))
        c, cb, s = jenks.quantize_gf4(W, 0)
        _same(pw, c, s, cb)


def test_rotated_packing_matches_oracle():
    rng = np.random.default_rng(5)
    W = (rng.standard_normal((6, 384)) * 0.02).astype(np.float32)
    pw = jq.pack_weight(torch.from_numpy(W), jq.QuantSpec("gf4", 128, 128))
    c, cb, s = jenks.quantize_gf4(formats.fwht_block(W, 128), 128)
    _same(pw, c, s, cb)


def test_golden_fixtures(golden_dir):
    z = np.load(os.path.join(golden_dir, "e2m1_g32.npz"))
    pw = jq.pack_weight(torch.from_numpy(z["W"]), jq.QuantSpec("e2m1", 32, 0))
    assert np.array_equal(pw.qweight.numpy(), z["qweight"])
    z = np.load(os.path.join(golden_dir, "gf4_g128_had.npz"))
    pw = jq.pack_weight(torch.from_numpy(z["W"]), jq.QuantSpec("gf4", 128, 128))
    assert np.array_equal(pw.qweight.numpy(), z["qweight"])
    assert np.array_equal(pw.codebook.numpy().view(np.uint16), z["codebook"].view(np.uint16))
    z = np.load(os.path.join(golden_dir, "lenet300_pruned_rows.npz"))
    pw = jq.pack_weight(torch.from_numpy(z["W"]), jq.QuantSpec("gf4", 0, 0))
    assert np.array_equal(pw.qweight.numpy(), z["qweight"])
    assert np.array_equal(pw.codebook.numpy().view(np.uint16), z["codebook"].view(np.uint16))


def test_golden_mlp_all_layers(golden_dir):
    """All three layers of the 784-300-100-10 model, including the 300x784
    one the O(k m^2) oracle is too slow to redo in the CPU suite: the
    committed hashes were produced by the oracle."""
    z = np.load(os.path.join(golden_dir, "mlp_gf4.npz"))
    g = torch.Generator("cpu").manual_seed(0)
    for li, (n, k) in enumerate([(300, 784), (100, 300), (10, 100)]):
        W = torch.randn(n, k, generator=g) * k ** -0.5
        pw = jq.pack_weight(W, jq.QuantSpec("gf4", 0, 0))
        assert hashlib.sha256(pw.qweight.numpy().tobytes()).hexdigest() == str(z[f"codes_sha{li}"])
        assert np.array_equal(pw.codebook.numpy().view(np.uint16), z[f"codebook{li}"].view(np.uint16))


def test_row_shards_are_slices():
    W = torch.randn(16, 256) * 0.02
    pw = jq.pack_weight(W, jq.QuantSpec("gf4", 128, 0))
    a, b = pw.rows(0, 8), pw.rows(8, 16)
    assert torch.equal(torch.cat([a.qweight, b.qweight]), pw.qweight)
    assert torch.equal(torch.cat([a.codebook, b.codebook]), pw.codebook)
    # every quantity is per row: packing a slice equals slicing the pack
    pa = jq.pack_weight(W[:8], jq.QuantSpec("gf4", 128, 0))
    assert torch.equal(pa.qweight, a.qweight) and torch.equal(pa.scales, a.scales)


# ------------------------------------------------------- pruned weights stay zero ----
def _host_dequant(pw):
    codes = formats.unpack_nibbles(pw.qweight.numpy(), pw.K)
    s = None if pw.scales is None else pw.scales.numpy()
    return formats.dequant_gf4(codes, pw.codebook.numpy(), s, pw.spec.group_size)


def test_pruned_checkpoint_zeros_survive_gf4(golden_dir):
    """All three layers of the reference's pruned LeNet-300-100 checkpoint
    (97.8 % zeros): the class that holds an exact zero carries the entry 0.0,
    so every pruned weight dequantises to exactly zero, as the reference's
    mask * s * (Q + Theta) does (Quantization_Experiments/layers.py:37,43)."""
    z = np.load(os.path.join(golden_dir, "lenet300_pruned_layers.npz"))
    for li in range(3):
        W = z[f"W{li}"]
        pw = jq.pack_weight(torch.from_numpy(W), jq.QuantSpec("gf4", 0, 0))
        assert hashlib.sha256(pw.qweight.numpy().tobytes()).hexdigest() == str(z[f"codes_sha{li}"])
        assert np.array_equal(pw.codebook.numpy().view(np.uint16), z[f"codebook{li}"].view(np.uint16))
        w_hat = _host_dequant(pw)
        assert np.all(w_hat[W == 0] == 0)
        assert np.all(np.diff(pw.codebook.numpy().astype(np.float32), axis=1) >= 0)


def test_zeros_survive_group_scaling(golden_dir):
    z = np.load(os.path.join(golden_dir, "gf4_sparse_g128.npz"))
    W = z["W"]
    pw = jq.pack_weight(torch.from_numpy(W), jq.QuantSpec("gf4", 128, 0))
    assert np.array_equal(pw.qweight.numpy(), z["qweight"])
    assert np.array_equal(pw.codebook.numpy().view(np.uint16), z["codebook"].view(np.uint16))
    assert np.array_equal(pw.scales.numpy().view(np.uint16), z["scales"].view(np.uint16))
    w_hat = _host_dequant(pw)
    assert np.array_equal(w_hat, z["w_hat"])
    assert np.all(w_hat[W == 0] == 0)


@pytest.mark.parametrize("g", [0, 128])
def test_a_few_zeros_per_row_stay_zero(g):
    """Lightly pruned rows: the zero would otherwise share a class with small
    non-zero neighbours and come back as their mean."""
    rng = np.random.default_rng(3)
    W = (rng.standard_normal((12, 512)) * 0.02).astype(np.float32)
    W[rng.random(W.shape) < 0.01] = 0.0
    W[0, 7] = -0.0
    pw = jq.pack_weight(torch.from_numpy(W), jq.QuantSpec("gf4", g, 0))
    c, cb, s = jenks.quantize_gf4(W, g)
    _same(pw, c, s, cb)
    w_hat = _host_dequant(pw)
    assert (W == 0).sum() > 20 and np.all(w_hat[W == 0] == 0)
    assert np.all(np.diff(cb.astype(np.float32), axis=1) >= 0)
