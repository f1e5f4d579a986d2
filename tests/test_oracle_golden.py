"""The CPU oracle against the committed golden vectors and known answers."""
import hashlib
import os

import numpy as np
import pytest

from oracle import formats, jenks


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_e2m1_byte_table(golden_dir):
    z = np.load(os.path.join(golden_dir, "kat_e2m1_bytes.npz"))
    codes = formats.unpack_nibbles(z["qweight"], 512)
    vals = formats.dequant_e2m1(codes, np.ones((1, 16), dtype=np.float16), 32)
    assert np.array_equal(vals, z["values"])
    # hand-checkable entries: byte 0x72 -> low nibble 2 (1.0), high nibble 7 (6.0)
    assert vals[0, 2 * 0x72] == 1.0 and vals[0, 2 * 0x72 + 1] == 6.0
    # byte 0x9f -> low nibble 0xf (-6.0), high nibble 9 (-0.5)
    assert vals[0, 2 * 0x9F] == -6.0 and vals[0, 2 * 0x9F + 1] == -0.5


def test_e2m1_rounding_rule():
    u = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, 100.0, -0.25, -0.75, -5.0, -9.0, 0.0, -0.0, 0.26],
                 dtype=np.float32)
    want = np.array([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, 6.0, 0.0, -1.0, -4.0, -6.0, 0.0, 0.0, 0.5])
    c = formats.e2m1_round_codes(u)
    assert np.array_equal(formats.E2M1_VALUES[c], want.astype(np.float32))
    assert not np.any(c == 8)  # negative zero is never emitted


def test_e2m1_scale_guards():
    W = np.zeros((2, 64), dtype=np.float32)
    W[1, :32] = 1e-9  # absmax/6 underflows fp16 -> scale 1.0
    c, s = formats.quantize_e2m1(W, 32)
    assert np.all(s == np.float16(1.0)) and np.all(c == 0)


def test_pack_unpack_roundtrip_ragged():
    rng = np.random.default_rng(0)
    for K in (1, 31, 32, 33, 100, 300, 784):
        c = rng.integers(0, 16, size=(3, K), dtype=np.uint8)
        q = formats.pack_nibbles(c)
        assert q.shape == (3, formats.row_stride_codes(K) // 2) and q.shape[1] % 16 == 0
        assert np.array_equal(formats.unpack_nibbles(q, K), c)


def test_fwht_unit_vectors_and_involution(golden_dir):
    rows = np.load(os.path.join(golden_dir, "kat_fwht128.npz"))["rows"]
    got = formats.fwht_block(np.eye(128, dtype=np.float32), 128)
    assert np.array_equal(got, rows)
    H = formats.hadamard_matrix(128) / np.sqrt(128.0)
    assert np.allclose(rows, H, atol=1e-7)
    x = np.random.default_rng(1).standard_normal((3, 384)).astype(np.float32)
    assert np.allclose(formats.fwht_block(formats.fwht_block(x)), x, atol=2e-6)
    # orthonormal: norms are preserved
    assert np.allclose(np.linalg.norm(formats.fwht_block(x), axis=1), np.linalg.norm(x, axis=1), rtol=1e-6)


@pytest.mark.parametrize("n,k", [(6, 2), (8, 3), (10, 4), (12, 5), (9, 16), (13, 6)])
def test_jenks_dp_equals_exhaustive(n, k):
    rng = np.random.default_rng(n * 100 + k)
    for _ in range(25):
        v = rng.standard_normal(n).astype(np.float32)
        a = jenks.jenks_breaks(v, k)[2]
        b = jenks.jenks_breaks(v, k, brute=True)[2]
        assert np.array_equal(a, b)


def test_jenks_two_classes_match_reference_form():
    rng = np.random.default_rng(7)
    for _ in range(40):
        v = np.sort(rng.standard_normal(48).astype(np.float32))
        br = jenks.jenks_breaks(v, 2)[2]
        assert br[1] == jenks.two_class_break_reference_form(v)


def test_jenks_fewer_distinct_values_than_classes():
    row = np.array([0, 0, 0, 0.5, 0.5, -1.0, 0, 0, 2.0, 0], dtype=np.float32)
    codes, cb = jenks.jenks_codebook_row(row, 16)
    assert np.array_equal(cb[:4], np.array([-1.0, 0.0, 0.5, 2.0], dtype=np.float16))
    assert np.all(cb[4:] == np.float16(2.0))
    assert np.array_equal(cb.astype(np.float32)[codes], row)  # lossless when distinct values <= 16


def test_hand_checkable_gf4_row():
    # two rows of 64: row 0 is 16 well-separated clusters of 4 equal values
    base = np.arange(16, dtype=np.float32) - 7.5
    W = np.stack([np.repeat(base, 4)[::-1].copy(), np.tile(np.array([-1, 1], dtype=np.float32), 32)])
    codes, cb, _ = jenks.quantize_gf4(W, 0)
    assert np.array_equal(cb[0].astype(np.float32), base)
    assert np.array_equal(codes[0], np.repeat(np.arange(16, dtype=np.uint8), 4)[::-1])
    assert np.array_equal(cb[1, :2].astype(np.float32), [-1, 1]) and np.all(cb[1, 2:] == 1)
    assert np.array_equal(formats.dequant_gf4(codes, cb, None, 0), W)


def test_golden_e2m1(golden_dir):
    z = np.load(os.path.join(golden_dir, "e2m1_g32.npz"))
    c, s = formats.quantize_e2m1(z["W"], 32)
    assert np.array_equal(formats.pack_nibbles(c), z["qweight"])
    assert np.array_equal(s.view(np.uint16), z["scales"].view(np.uint16))
    w_hat = formats.dequant_e2m1(formats.unpack_nibbles(z["qweight"], 256), z["scales"], 32)
    assert np.array_equal(w_hat, z["w_hat"])
    y = formats.linear_ref(z["x"], w_hat, z["bias"])
    assert formats.rel_err(y, z["y"]) < 2e-6  # reference F.linear sums in fp32


def test_golden_gf4_hadamard(golden_dir):
    z = np.load(os.path.join(golden_dir, "gf4_g128_had.npz"))
    c, cb, s = jenks.quantize_gf4(formats.fwht_block(z["W"], 128), 128)
    assert np.array_equal(formats.pack_nibbles(c), z["qweight"])
    assert np.array_equal(cb.view(np.uint16), z["codebook"].view(np.uint16))
    assert np.array_equal(s.view(np.uint16), z["scales"].view(np.uint16))
    assert np.array_equal(formats.fwht_block(z["x"], 128), z["x_rot"])
    y = formats.linear_ref(z["x"], z["w_hat"], None, had_block=128)
    assert formats.rel_err(y, z["y"]) < 2e-6
    # the rotation is orthonormal: rotating both sides leaves W x unchanged (up to fp32 rounding)
    y_plain = z["x"].astype(np.float64) @ z["W"].astype(np.float64).T
    y_rot = z["x_rot"].astype(np.float64) @ formats.fwht_block(z["W"], 128).astype(np.float64).T
    assert formats.rel_err(y_rot, y_plain) < 1e-5


def test_golden_mlp(golden_dir):
    z = np.load(os.path.join(golden_dir, "mlp_gf4.npz"))
    import torch
    g = torch.Generator("cpu").manual_seed(0)
    dims = [(300, 784), (100, 300), (10, 100)]
    Ws = [(torch.randn(n, k, generator=g) * k ** -0.5).numpy() for n, k in dims]
    x = torch.rand(1, 784, generator=g).numpy()
    assert np.array_equal(x, z["x"])
    h = x
    for li, W in enumerate(Ws[1:], start=1):  # layer 0 (300x784 at O(k m^2)) is covered by the packer test
        pass
    for li in (1, 2):
        c, cb, _ = jenks.quantize_gf4(Ws[li], 0)
        assert np.array_equal(cb.view(np.uint16), z[f"codebook{li}"].view(np.uint16))
        assert _sha(formats.pack_nibbles(c)) == str(z[f"codes_sha{li}"])
        w_hat = formats.dequant_gf4(c, cb, None, 0)
        assert _sha(w_hat) == str(z[f"what_sha{li}"])
        h_in = np.maximum(z[f"y{li - 1}"], 0)
        assert formats.rel_err(formats.linear_ref(h_in, w_hat, None), z[f"y{li}"]) < 2e-6


def test_golden_pruned_checkpoint_rows(golden_dir):
    z = np.load(os.path.join(golden_dir, "lenet300_pruned_rows.npz"))
    c, cb, _ = jenks.quantize_gf4(z["W"], 0)
    assert np.array_equal(formats.pack_nibbles(c), z["qweight"])
    assert np.array_equal(cb.view(np.uint16), z["codebook"].view(np.uint16))
    w_hat = formats.dequant_gf4(c, cb, None, 0)
    assert formats.rel_err(formats.linear_ref(z["x"], w_hat, None), z["y"]) < 2e-6
    assert (z["W"] == 0).mean() > 0.9  # the fixture really is sparse


def test_activation_model_is_tight():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 512)).astype(np.float32) * np.array([[1e-6], [3e4]], dtype=np.float32)
    m = formats.activation_fp16_model(x, had=False)
    assert np.max(np.abs(m - x) / np.abs(x).max(axis=1, keepdims=True)) < 2.0 ** -11
