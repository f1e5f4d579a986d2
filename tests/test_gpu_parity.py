"""CUDA path vs the CPU oracle, through the C ABI.  Integer / byte results
(unpacked codes, dequantized weights, the fp32 rotation) must be bit-exact;
GEMV outputs must satisfy  max|y - y_ref| / max|y_ref| <= 1e-3  against the
fp32 oracle on identical inputs (TOL below), and a much tighter bound against
the oracle that also models the kernel's fp16 rounding of the activation."""
import os

import numpy as np
import pytest
import torch

import if_i_could_turn_back_time_b200 as jq
from if_i_could_turn_back_time_b200 import ops
from oracle import formats

pytestmark = pytest.mark.gpu
TOL = 1e-3          # the parity gate
TOL_MODEL = 3e-6    # same arithmetic, only the fp32 summation order differs
TOL_FOLDED = 5e-5   # tensor-memory kernel, E2M1: fp16 weights with the group scale folded in; the tensor core's fp32
                    # accumulation over K up to 28672 is a little looser than a chain of fp32 FMAs
DEV = "cuda:0"


def _oracle_dequant(pw):
    codes = formats.unpack_nibbles(pw.qweight.cpu().numpy(), pw.K)
    s = None if pw.scales is None else pw.scales.cpu().numpy()
    if pw.spec.fmt == "e2m1":
        return formats.dequant_e2m1(codes, s, pw.spec.group_size)
    return formats.dequant_gf4(codes, pw.codebook.cpu().numpy(), s, pw.spec.group_size)


def _weights(N, K, seed, outliers=True):
    g = torch.Generator("cpu").manual_seed(seed)
    W = torch.randn(N, K, generator=g) * 0.02
    if outliers:
        W[torch.rand(N, K, generator=g) < 0.001] *= 10
    return W


def _check_gemv(pw, x_cpu, bias_cpu=None):
    """x_cpu: torch tensor [B,K] of the activation dtype."""
    pwd = pw.to(DEV)
    w_hat = _oracle_dequant(pw)
    x32 = x_cpu.float().numpy()
    b32 = None if bias_cpu is None else bias_cpu.numpy()
    y = ops.linear(x_cpu.to(DEV), pwd, None if bias_cpu is None else bias_cpu.to(DEV), out_dtype=torch.float32)
    y = y.cpu().numpy()
    ref = formats.linear_ref(x32, w_hat, b32, had_block=pw.spec.had_block)
    err = formats.rel_err(y, ref)
    assert err <= TOL, f"rel err {err:.3e} vs fp32 oracle"
    xm = formats.activation_fp16_model(x32, had=bool(pw.spec.had_block))
    tol_m = TOL_MODEL
    if pw.spec.fmt == "e2m1" and ops.ta_eligible(pw.spec.fmt_id, pw.K, pw.spec.group_size, x_cpu.shape[0]):
        # the tensor-memory kernel multiplies the E2M1 value by the group's fp16 scale in fp16 (one rounding)
        codes = formats.unpack_nibbles(pw.qweight.cpu().numpy(), pw.K)
        w_hat = formats.dequant_e2m1_folded_fp16(codes, pw.scales.cpu().numpy(), pw.spec.group_size)
        tol_m = TOL_FOLDED
    ref_m = formats.linear_ref(xm, w_hat, b32)
    err_m = formats.rel_err(y, ref_m)
    assert err_m <= tol_m, f"rel err {err_m:.3e} vs the model of the kernel's arithmetic"
    assert ops.check_status(raise_on_error=False) == 0, "a device-side wait timed out"
    return err


# ---------------------------------------------------------------- dequant ----
def test_dequant_e2m1_every_byte(golden_dir):
    z = np.load(os.path.join(golden_dir, "kat_e2m1_bytes.npz"))
    pw = jq.PackedWeight(jq.QuantSpec("e2m1", 32, 0), 1, 512, torch.from_numpy(z["qweight"]),
                         torch.ones(1, 16, dtype=torch.float16), None).to(DEV)
    got = ops.dequantize(pw).cpu().numpy()
    assert np.array_equal(got, z["values"])
    assert np.array_equal(np.signbit(got), np.signbit(z["values"]))  # code 8 is -0.0


@pytest.mark.parametrize("fmt,N,K,g", [("e2m1", 64, 256, 32), ("e2m1", 33, 4096, 32), ("e2m1", 7, 192, 64),
                                        ("gf4", 48, 1024, 128), ("gf4", 5, 784, 0), ("gf4", 9, 300, 0),
                                        ("gf4", 3, 100, 0), ("gf4", 17, 512, 64)])
def test_dequant_bit_exact(fmt, N, K, g):
    pw = jq.pack_weight(_weights(N, K, N + K), jq.QuantSpec(fmt, g, 0))
    got = ops.dequantize(pw.to(DEV)).cpu().numpy()
    assert np.array_equal(got, _oracle_dequant(pw))


def test_dequant_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "e2m1_g32.npz"))
    pw = jq.PackedWeight(jq.QuantSpec("e2m1", 32, 0), 64, 256, torch.from_numpy(z["qweight"]),
                         torch.from_numpy(z["scales"]), None).to(DEV)
    assert np.array_equal(ops.dequantize(pw).cpu().numpy(), z["w_hat"])
    z = np.load(os.path.join(golden_dir, "gf4_g128_had.npz"))
    pw = jq.PackedWeight(jq.QuantSpec("gf4", 128, 128), 32, 512, torch.from_numpy(z["qweight"]),
                         torch.from_numpy(z["scales"]), torch.from_numpy(z["codebook"])).to(DEV)
    assert np.array_equal(ops.dequantize(pw).cpu().numpy(), z["w_hat"])


# ------------------------------------------------------------------- fwht ----
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_fwht_bit_exact(dtype, golden_dir):
    g = torch.Generator("cpu").manual_seed(3)
    x = (torch.randn(5, 1024, generator=g) * 3).to(dtype)
    got = ops.fwht_block(x.to(DEV)).cpu().numpy()
    assert np.array_equal(got, formats.fwht_block(x.float().numpy(), 128))
    rows = np.load(os.path.join(golden_dir, "kat_fwht128.npz"))["rows"]
    assert np.array_equal(ops.fwht_block(torch.eye(128, device=DEV)).cpu().numpy(), rows)


# ------------------------------------------------------------------- gemv ----
@pytest.mark.parametrize("B", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("fmt,g,had", [("e2m1", 32, 0), ("gf4", 128, 128), ("gf4", 128, 0), ("e2m1", 64, 128)])
def test_gemv_parity_batches(fmt, g, had, B):
    pw = jq.pack_weight(_weights(203, 1024, 17), jq.QuantSpec(fmt, g, had))
    gen = torch.Generator("cpu").manual_seed(B)
    x = torch.randn(B, 1024, generator=gen).bfloat16()
    _check_gemv(pw, x)


@pytest.mark.parametrize("N,K,fmt,g,had", [(1, 128, "e2m1", 32, 128), (2, 32, "e2m1", 32, 0), (5, 64, "gf4", 0, 0),
                                            (300, 784, "gf4", 0, 0), (100, 300, "gf4", 0, 0), (10, 100, "gf4", 0, 0),
                                            (67, 2048 + 128, "gf4", 128, 128), (129, 11008, "gf4", 128, 128),
                                            (64, 28672, "e2m1", 32, 0), (4099, 256, "e2m1", 32, 0)])
def test_gemv_parity_shapes(N, K, fmt, g, had):
    pw = jq.pack_weight(_weights(N, K, N * 7 + K), jq.QuantSpec(fmt, g, had))
    gen = torch.Generator("cpu").manual_seed(N)
    _check_gemv(pw, torch.rand(1, K, generator=gen), torch.randn(N, generator=gen))
    _check_gemv(pw, torch.randn(2, K, generator=gen).half())


@pytest.mark.parametrize("N,K,had", [(16, 256, 0), (5, 256, 128), (203, 1024, 0), (48, 2048, 128), (33, 11008, 0),
                                     (1000, 4096, 128), (17, 8192, 0)])
@pytest.mark.parametrize("B", [2, 3, 7, 8])
def test_e2m1_batched_rows_on_the_mma_loop(N, K, had, B):
    """E2M1 g32, K a multiple of 256, batch 2..8: the m16n8k16 row loop, with one, two or four K parts per
    row group (K = 256 / 1024 / 2048+), ragged N, rotation on and off."""
    pw = jq.pack_weight(_weights(N, K, N + 3 * K), jq.QuantSpec("e2m1", 32, had))
    gen = torch.Generator("cpu").manual_seed(N + B)
    _check_gemv(pw, torch.randn(B, K, generator=gen).bfloat16(), torch.randn(N, generator=gen))


@pytest.mark.parametrize("N,K,had", [(16, 256, 0), (5, 256, 128), (203, 1024, 128), (48, 2048, 0), (33, 11008, 128),
                                     (1000, 4096, 128)])
@pytest.mark.parametrize("B", [2, 3, 7, 8])
def test_gf4_batched_rows_on_the_mma_loop(N, K, had, B):
    """GF4 g128, K a multiple of 256, batch 2..8: per-lane table columns feeding the m16n8k16 row loop."""
    pw = jq.pack_weight(_weights(N, K, N + 5 * K), jq.QuantSpec("gf4", 128, had))
    gen = torch.Generator("cpu").manual_seed(N + B)
    _check_gemv(pw, torch.randn(B, K, generator=gen).bfloat16(), torch.randn(N, generator=gen))
    # a row shard sums in the same order as the whole matrix
    if N >= 48:
        pwd = pw.to(DEV)
        x = torch.randn(B, K, generator=gen).bfloat16().to(DEV)
        y = ops.linear(x, pwd, out_dtype=torch.float32)
        assert torch.equal(ops.linear(x, pwd.rows(16, 48), out_dtype=torch.float32), y[:, 16:48])


def test_gf4_grouped_launch_tiles_k():
    shapes = [(200, 11008), (64, 4096), (33, 256)]
    pws = [jq.pack_weight(_weights(n, k, n + k), jq.QuantSpec("gf4", 128, 128)).to(DEV) for n, k in shapes]
    gen = torch.Generator("cpu").manual_seed(3)
    grp = ops.GroupedGemv(pws, 8, torch.float32)
    for x in grp.xs:
        x.copy_(torch.randn(x.shape, generator=gen))
    grp.run()
    torch.cuda.synchronize()
    assert grp.launches_per_run == 1
    for pw, x, y in zip(pws, grp.xs, grp.ys):
        assert formats.rel_err(y.cpu().numpy(), ops.linear(x, pw).cpu().numpy()) <= 2e-6


def test_e2m1_batched_fallbacks_and_row_shards_agree_bit_for_bit():
    gen = torch.Generator("cpu").manual_seed(9)
    # not eligible for the MMA loop (K % 256 != 0, or 64-code groups): the FMA loops take them
    for K, g in ((1152, 32), (1024, 64)):
        pw = jq.pack_weight(_weights(70, K, K), jq.QuantSpec("e2m1", g, 0))
        _check_gemv(pw, torch.randn(5, K, generator=gen).half())
    # a row shard computes exactly what the whole matrix computes for those rows (same summation order)
    pw = jq.pack_weight(_weights(320, 4096, 5), jq.QuantSpec("e2m1", 32, 128)).to(DEV)
    x = torch.randn(6, 4096, generator=gen).bfloat16().to(DEV)
    y = ops.linear(x, pw, out_dtype=torch.float32)
    for lo, hi in ((0, 160), (160, 320), (37, 90)):
        assert torch.equal(ops.linear(x, pw.rows(lo, hi), out_dtype=torch.float32), y[:, lo:hi])
    # unit vectors: exact columns of the dequantised matrix, every batch row its own column
    w_hat = ops.dequantize(pw)
    ks = [0, 1, 31, 32, 255, 256, 4095]
    xe = torch.zeros(len(ks), 4096, device=DEV)
    for i, k in enumerate(ks):
        xe[i, k] = 1.0
    pw0 = jq.pack_weight(_weights(320, 4096, 5), jq.QuantSpec("e2m1", 32, 0)).to(DEV)
    assert torch.equal(ops.linear(xe, pw0), ops.dequantize(pw0)[:, ks].t().contiguous())


def test_gemv_heavy_tailed_activations_and_extreme_magnitudes():
    K = 4096
    pw = jq.pack_weight(_weights(256, K, 2), jq.QuantSpec("gf4", 128, 128))
    g = torch.Generator("cpu").manual_seed(2)
    z = torch.randn(5, 1, K, generator=g)
    x = z[0] / torch.sqrt((z[1:] ** 2).mean(dim=0))
    x[:, torch.randperm(K, generator=g)[:8]] *= 50
    _check_gemv(pw, x.bfloat16())
    for scale in (1e-20, 1e-6, 1e8, 1e25):
        _check_gemv(pw, (x * scale).float())
    y0 = ops.linear(torch.zeros(1, K, device=DEV), pw.to(DEV))
    assert torch.count_nonzero(y0) == 0


def test_gemv_unit_vectors_read_back_dequantized_columns():
    """x = e_k is exact in fp16, so y must equal column k of W_hat bit for bit."""
    pw = jq.pack_weight(_weights(512, 1024, 4), jq.QuantSpec("e2m1", 32, 0)).to(DEV)
    w_hat = ops.dequantize(pw)
    for k in (0, 1, 31, 32, 517, 1023):
        x = torch.zeros(1, 1024, device=DEV)
        x[0, k] = 1.0
        assert torch.equal(ops.linear(x, pw)[0], w_hat[:, k])


def test_output_dtypes_round_once():
    pw = jq.pack_weight(_weights(128, 512, 6), jq.QuantSpec("e2m1", 32, 0)).to(DEV)
    x = torch.randn(3, 512, generator=torch.Generator("cpu").manual_seed(1)).bfloat16().to(DEV)
    y32 = ops.linear(x, pw, out_dtype=torch.float32)
    assert torch.equal(ops.linear(x, pw), y32.bfloat16())
    assert torch.equal(ops.linear(x.half(), pw), ops.linear(x.half(), pw, out_dtype=torch.float32).half())


def test_golden_vectors_through_the_kernel(golden_dir):
    z = np.load(os.path.join(golden_dir, "e2m1_g32.npz"))
    pw = jq.PackedWeight(jq.QuantSpec("e2m1", 32, 0), 64, 256, torch.from_numpy(z["qweight"]),
                         torch.from_numpy(z["scales"]), None).to(DEV)
    y = ops.linear(torch.from_numpy(z["x"]).bfloat16().to(DEV), pw, torch.from_numpy(z["bias"]).to(DEV),
                   out_dtype=torch.float32)
    assert formats.rel_err(y.cpu().numpy(), z["y"]) <= TOL
    z = np.load(os.path.join(golden_dir, "gf4_g128_had.npz"))
    pw = jq.PackedWeight(jq.QuantSpec("gf4", 128, 128), 32, 512, torch.from_numpy(z["qweight"]),
                         torch.from_numpy(z["scales"]), torch.from_numpy(z["codebook"])).to(DEV)
    y = ops.linear(torch.from_numpy(z["x"]).bfloat16().to(DEV), pw, out_dtype=torch.float32)
    assert formats.rel_err(y.cpu().numpy(), z["y"]) <= TOL
    z = np.load(os.path.join(golden_dir, "lenet300_pruned_rows.npz"))
    pw = jq.PackedWeight(jq.QuantSpec("gf4", 0, 0), 24, 784, torch.from_numpy(z["qweight"]), None,
                         torch.from_numpy(z["codebook"])).to(DEV)
    y = ops.linear(torch.from_numpy(z["x"]).to(DEV), pw)
    assert formats.rel_err(y.cpu().numpy(), z["y"]) <= TOL


def test_mlp_784_300_100_10_matches_golden(golden_dir):
    """The reference's model container (Flatten, Linear, ReLU, Linear, ReLU,
    Linear) with every Linear swapped by quantize_module."""
    z = np.load(os.path.join(golden_dir, "mlp_gf4.npz"))
    g = torch.Generator("cpu").manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(784, 300, bias=False), torch.nn.ReLU(),
                                torch.nn.Linear(300, 100, bias=False), torch.nn.ReLU(),
                                torch.nn.Linear(100, 10, bias=False))
    with torch.no_grad():
        for idx, (n, k) in zip((1, 3, 5), [(300, 784), (100, 300), (10, 100)]):
            model[idx].weight.copy_(torch.randn(n, k, generator=g) * k ** -0.5)
    qm = jq.quantize_module(model, 4, fmt="gf4", group_size=0).to(DEV)
    x = torch.from_numpy(z["x"]).to(DEV)
    y = qm(x)
    assert formats.rel_err(y.cpu().numpy(), z["y2"]) <= TOL
    h = qm[1](x)
    assert formats.rel_err(h.cpu().numpy(), z["y0"]) <= TOL
    # commit() drops the dense weight; .weight stays readable as W_hat
    qm[1].commit()
    assert qm[1].hard_quant and torch.equal(qm[1](x), h)
    assert qm[1].weight.shape == (300, 784) and qm[1].weight.dtype == torch.float32


def test_leading_dims_and_large_batch_split():
    pw = jq.pack_weight(_weights(96, 256, 8), jq.QuantSpec("e2m1", 32, 0)).to(DEV)
    x = torch.randn(3, 7, 256, generator=torch.Generator("cpu").manual_seed(0)).to(DEV)
    y = ops.linear(x, pw)
    assert y.shape == (3, 7, 96)
    y1 = torch.cat([ops.linear(x.reshape(21, 256)[i:i + 1], pw) for i in range(21)])
    # 21 rows go through the tensor-core kernel (E4M3-term activation), single rows through the GEMV
    # (fp16 activation): both are within the gate of the oracle, hence within 2x of each other
    assert formats.rel_err(y.reshape(21, 96).cpu().numpy(), y1.cpu().numpy()) < 2 * TOL


def test_split_k_large_batch_times_k():
    """B x K too large to stage in shared memory: runs as split-K through a
    caller workspace of fp32 partials; must agree with the oracle and with the
    workspace-free sub-batch path."""
    from if_i_could_turn_back_time_b200 import _lib
    lib = _lib.load()
    N, K, B = 96, 28672, 8
    assert lib.jq_workspace_bytes(0, N, K, B) > 0 and lib.jq_workspace_bytes(0, N, 4096, 1) == 0
    for fmt, g in (("e2m1", 32), ("gf4", 128)):
        pw = jq.pack_weight(_weights(N, K, 5), jq.QuantSpec(fmt, g, 128))
        gen = torch.Generator("cpu").manual_seed(3)
        x = torch.randn(B, K, generator=gen).bfloat16()
        bias = torch.randn(N, generator=gen)
        _check_gemv(pw, x, bias)
        pwd, xd, bd = pw.to(DEV), x.to(DEV), bias.to(DEV)
        y_ws = ops.linear(xd, pwd, bd, out_dtype=torch.float32)
        y_sub = torch.cat([ops.linear(xd[i:i + 2], pwd, bd, out_dtype=torch.float32) for i in range(0, B, 2)])
        assert formats.rel_err(y_ws.cpu().numpy(), y_sub.cpu().numpy()) < 2e-6


# --------------------------------------------------- batches above 8 rows ----
def _random_packed(fmt, N, K, g, had, seed):
    """Packed tensors drawn directly (every code equally likely, scales around the size a packer would give):
    full-size matrices without the cost of packing them."""
    rng = np.random.default_rng(seed)
    qw = torch.from_numpy(rng.integers(0, 256, (N, K // 2), dtype=np.uint8))
    sc = torch.from_numpy((0.01 * (0.5 + rng.random((N, K // g), dtype=np.float32))).astype(np.float16))
    cb = None
    if fmt == "gf4":
        cb = torch.from_numpy(np.sort(rng.standard_normal((N, 16), dtype=np.float32), axis=1).astype(np.float16))
    return jq.PackedWeight(jq.QuantSpec(fmt, g, had), N, K, qw, sc, cb)


def _check_rows(pw, x_cpu, rows, bias_cpu=None):
    """Full-size matrix, oracle on a sample of its rows (every output row is an independent dot product)."""
    pwd = pw.to(DEV)
    y = ops.linear(x_cpu.to(DEV), pwd, None if bias_cpu is None else bias_cpu.to(DEV), out_dtype=torch.float32)
    assert ops.check_status(raise_on_error=False) == 0
    y = y.cpu().numpy()
    assert np.isfinite(y).all()
    rows = np.asarray(rows)
    sub = jq.PackedWeight(pw.spec, len(rows), pw.K, pw.qweight[rows], pw.scales[rows],
                          None if pw.codebook is None else pw.codebook[rows])
    ref = formats.linear_ref(x_cpu.float().numpy(), _oracle_dequant(sub),
                             None if bias_cpu is None else bias_cpu.numpy()[rows], had_block=pw.spec.had_block)
    scale = np.abs(ref).max()
    assert np.abs(y[:, rows] - ref).max() / scale <= TOL
    return y


@pytest.mark.parametrize("B", [9, 16, 17, 32, 33, 64, 128])
@pytest.mark.parametrize("fmt,g,had", [("e2m1", 32, 0), ("gf4", 128, 128)])
def test_batches_above_eight_rows(fmt, g, had, B):
    """9..64 rows in one pass of the tensor-memory kernel (GF4: 16 rows per pass), more in several passes."""
    pw = jq.pack_weight(_weights(300, 1024, 21), jq.QuantSpec(fmt, g, had))
    assert ops.ta_eligible(pw.spec.fmt_id, 1024, g, B)
    gen = torch.Generator("cpu").manual_seed(B)
    _check_gemv(pw, torch.randn(B, 1024, generator=gen).bfloat16(), torch.randn(300, generator=gen))


@pytest.mark.parametrize("N,K,had,dtype", [(128, 512, 0, torch.bfloat16), (1, 512, 128, torch.bfloat16),
                                            (257, 4096, 0, torch.float32), (4096, 4096, 0, torch.bfloat16),
                                            (1024, 8192, 128, torch.float16), (130, 28672, 128, torch.bfloat16)])
@pytest.mark.parametrize("fmt,g", [("e2m1", 32), ("gf4", 128)])
def test_tensor_memory_kernel_shapes(fmt, g, N, K, had, dtype):
    pw = jq.pack_weight(_weights(N, K, N + K), jq.QuantSpec(fmt, g, had))
    gen = torch.Generator("cpu").manual_seed(N)
    _check_gemv(pw, torch.randn(16, K, generator=gen).to(dtype))
    _check_gemv(pw, (torch.randn(40, K, generator=gen) * 1e-4).to(dtype), torch.randn(N, generator=gen) * 1e-4)


def test_k_256_stays_on_the_row_loops_at_every_batch():
    """The TMA-fed kernels need K >= 512; shorter rows run as sub-batches of 8 on the row loops."""
    for fmt, g in (("e2m1", 32), ("gf4", 128)):
        pw = jq.pack_weight(_weights(70, 256, 9), jq.QuantSpec(fmt, g, 128))
        assert not ops.ta_eligible(pw.spec.fmt_id, 256, g, 24)
        _check_gemv(pw, torch.randn(24, 256, generator=torch.Generator("cpu").manual_seed(1)).bfloat16())


def test_misaligned_scales_fall_back_to_the_row_loops_and_misaligned_codebooks_are_refused():
    """E2M1 scales that start 8 bytes into an allocation cannot be read in 16-byte pieces by the tensor-memory
    kernel; the row loops (2-byte alignment) serve the call.  A codebook that is not 16-byte aligned is refused
    before any launch: every kernel fetches codebook rows with 16-byte copies."""
    from if_i_could_turn_back_time_b200 import _lib

    def shifted(t):
        raw = torch.empty(t.numel() * t.element_size() + 8, dtype=torch.uint8, device=DEV)
        v = raw[8:].view(t.dtype).view(t.shape)
        v.copy_(t)
        return v

    pw = jq.pack_weight(_weights(64, 1024, 4), jq.QuantSpec("e2m1", 32, 0)).to(DEV)
    off = jq.PackedWeight(pw.spec, pw.N, pw.K, pw.qweight, shifted(pw.scales), None)
    assert off.scales.data_ptr() % 16 == 8
    x = torch.randn(16, 1024, generator=torch.Generator("cpu").manual_seed(3)).bfloat16().to(DEV)
    y = ops.linear(x, off, out_dtype=torch.float32)
    y_rows = torch.cat([ops.linear(x[i:i + 8], pw, out_dtype=torch.float32) for i in range(0, 16, 8)])
    # both went through the row loops (the aligned one on the mma.sync loop, the other on the FMA loop): same
    # weights and activation rounding, fp32 summation order differs
    assert formats.rel_err(y.cpu().numpy(), y_rows.cpu().numpy()) <= 1e-5

    pg = jq.pack_weight(_weights(64, 1024, 4), jq.QuantSpec("gf4", 128, 128)).to(DEV)
    bad = jq.PackedWeight(pg.spec, pg.N, pg.K, pg.qweight, pg.scales, shifted(pg.codebook))
    for rows in (1, 4, 16):
        with pytest.raises(_lib.JqError):
            ops.linear(x[:rows], bad)
    torch.cuda.synchronize()                                         # nothing was launched, the context is healthy


@pytest.mark.parametrize("fmt,g,had,B", [("gf4", 128, 128, 1), ("gf4", 128, 128, 16), ("e2m1", 32, 0, 1), ("e2m1", 32, 0, 16)])
def test_linear_replays_from_a_cuda_graph(fmt, g, had, B):
    """After one warm-up call on the capture stream (which allocates that stream's scratch) a call enqueues
    kernels only: it can be captured and replayed with new inputs."""
    pw = jq.pack_weight(_weights(192, 1024, 12), jq.QuantSpec(fmt, g, had)).to(DEV)
    gen = torch.Generator("cpu").manual_seed(B)
    x = torch.randn(B, 1024, generator=gen).bfloat16().to(DEV)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ops.linear(x, pw)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        y = ops.linear(x, pw)
    x2 = torch.randn(B, 1024, generator=gen).bfloat16().to(DEV)
    x.copy_(x2)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, ops.linear(x2, pw))


def test_large_batch_is_split_and_matches_the_row_loops():
    pw = jq.pack_weight(_weights(512, 1024, 3), jq.QuantSpec("e2m1", 32, 0)).to(DEV)
    x = torch.randn(130, 1024, generator=torch.Generator("cpu").manual_seed(2)).bfloat16().to(DEV)
    y_ta = ops.linear(x, pw, out_dtype=torch.float32)
    assert ops.check_status(raise_on_error=False) == 0
    y_cc = torch.cat([ops.linear(x[i:i + 8], pw, out_dtype=torch.float32) for i in range(0, 130, 8)])
    # same activation rounding; the weights differ by the one fp16 rounding of value x scale
    assert formats.rel_err(y_ta.cpu().numpy(), y_cc.cpu().numpy()) <= TOL


@pytest.mark.parametrize("N,K", [(8192, 8192), (28672, 8192), (8192, 28672)])
@pytest.mark.parametrize("B", [1, 8, 32])
def test_e2m1_at_the_largest_configured_sizes(N, K, B):
    """The 70B-class projection shapes, E2M1 g32 with the rotation: batch 1 and 8 on the row loops (K = 28672 at
    batch 8 through the split-K scratch), 32 on the tensor-memory kernel."""
    pw = _random_packed("e2m1", N, K, 32, 128, N + K)
    gen = torch.Generator("cpu").manual_seed(B)
    rows = np.concatenate([np.arange(0, 130), np.arange(N // 2 - 3, N // 2 + 130), np.arange(N - 129, N)])
    _check_rows(pw, torch.randn(B, K, generator=gen).bfloat16(), rows, torch.randn(N, generator=gen))


@pytest.mark.parametrize("B", [1, 8, 16])
def test_gf4_at_the_largest_configured_sizes(B):
    pw = _random_packed("gf4", 28672, 8192, 128, 128, 77)
    gen = torch.Generator("cpu").manual_seed(B)
    rows = np.concatenate([np.arange(0, 70), np.arange(14000, 14200), np.arange(28672 - 65, 28672)])
    _check_rows(pw, torch.randn(B, 8192, generator=gen).bfloat16(), rows)


@pytest.mark.parametrize("fmt,g,B", [("e2m1", 32, 1), ("e2m1", 32, 32), ("gf4", 128, 1), ("gf4", 128, 8)])
def test_grouped_launch_at_70b_layer_shapes(fmt, g, B):
    """One transformer layer of the 70B-class workload (q/o 8192x8192, k/v 1024x8192, gate/up 28672x8192, down
    8192x28672) as one grouped launch; every matrix against the oracle on sampled rows, and bit for bit
    against the single-matrix call."""
    shapes = [(8192, 8192), (1024, 8192), (1024, 8192), (8192, 8192), (28672, 8192), (28672, 8192), (8192, 28672)]
    pws = [_random_packed(fmt, n, k, g, 128, 11 * i + n) for i, (n, k) in enumerate(shapes)]
    pwd = [p.to(DEV) for p in pws]
    grp = ops.GroupedGemv(pwd, B, torch.bfloat16)
    gen = torch.Generator("cpu").manual_seed(B)
    for x in grp.xs:
        x.copy_(torch.randn(x.shape, generator=gen).bfloat16())
    grp.run()
    assert grp.status() == 0
    for pw, x, y in zip(pws, grp.xs, grp.ys):
        rows = np.concatenate([np.arange(0, 64), np.arange(pw.N - 64, pw.N)])
        sub = jq.PackedWeight(pw.spec, len(rows), pw.K, pw.qweight[rows], pw.scales[rows],
                              None if pw.codebook is None else pw.codebook[rows])
        ref = formats.linear_ref(x.float().cpu().numpy(), _oracle_dequant(sub), None, had_block=128)
        got = y.float().cpu().numpy()[:, rows]
        assert np.abs(got - ref).max() / np.abs(ref).max() <= 2.0 ** -8 + TOL   # bf16 outputs


def test_bounded_wait_gives_up_with_a_status_and_the_device_stays_usable():
    """Failure path of the pipeline's waits, exercised without a fault: a wait on a barrier that nothing
    signals runs out after a bounded number of polls, the kernel reports JQ_ERR_TIMEOUT and returns."""
    import ctypes
    from if_i_could_turn_back_time_b200 import _lib
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = lib.jq_selftest_bounded_wait(ctypes.c_void_p(status.data_ptr()), 4096,
                                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0
    torch.cuda.synchronize()
    assert int(status.item()) == -7 and "wait" in _lib.strerror(-7)
    # the context is still healthy: a normal call right after works
    pw = jq.pack_weight(_weights(64, 256, 1), jq.QuantSpec("e2m1", 32, 0)).to(DEV)
    assert torch.isfinite(ops.linear(torch.randn(16, 256, device=DEV).bfloat16(), pw).float()).all()
    pw = jq.pack_weight(_weights(64, 512, 1), jq.QuantSpec("e2m1", 32, 0)).to(DEV)
    assert torch.isfinite(ops.linear(torch.randn(16, 512, device=DEV).bfloat16(), pw).float()).all()
    assert ops.check_status(raise_on_error=False) == 0


def test_grouped_batched_layers_equal_single_calls():
    shapes = [(512, 1024), (96, 2048), (300, 512)]
    pws = [jq.pack_weight(_weights(n, k, n + k), jq.QuantSpec("e2m1", 32, 0)).to(DEV) for n, k in shapes]
    grp = ops.GroupedGemv(pws, 24, torch.bfloat16)
    gen = torch.Generator("cpu").manual_seed(5)
    for x in grp.xs:
        x.copy_(torch.randn(x.shape, generator=gen).bfloat16())
    grp.run()
    assert grp.status() == 0
    for pw, x, y in zip(pws, grp.xs, grp.ys):
        assert torch.equal(y, ops.linear(x, pw))


# ------------------------------------------------------- BRECQ boundary ----
def test_replace_forward_boundary_with_a_weight_quantizer(golden_dir):
    """A Linear whose forward the reference's replace_forward has swapped for
    F.linear(x, module.weight_quantizer(), bias) (Quantization_Experiments/brecq.py:321-329), with a converged
    AdaRoundQuantizer (brecq.py:59-92) on a 4-bit per-row grid and pruned entries masked to zero.  The fixture
    holds W_q and the outputs of the reference's own code; the packed forward must reproduce them."""
    from if_i_could_turn_back_time_b200.linear import attach_packed_forward
    z = np.load(os.path.join(golden_dir, "brecq_replace_forward.npz"))
    lin = torch.nn.Linear(256, 48).to(DEV)
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(z["W"]))
        lin.bias.copy_(torch.from_numpy(z["bias"]))
    w_q = torch.from_numpy(z["W_q"]).to(DEV)
    attach_packed_forward(lin, lambda: w_q)
    assert torch.equal(lin.weight_quantizer(), w_q)                   # calibration code still sees the dense W_q
    w_hat = ops.dequantize(lin.packed_weight).cpu().numpy()
    assert np.all(w_hat[z["W_q"] == 0] == 0)                          # AdaRound's mask survives packing
    # at most 16 levels per row: every level is its own class, the codebook holds fp16(level)
    assert np.abs(w_hat - z["W_q"]).max() <= 2.0 ** -11 * np.abs(z["W_q"]).max()
    y = lin(torch.from_numpy(z["x"]).to(DEV)).detach().cpu().numpy()
    assert formats.rel_err(y, z["y"]) <= TOL


def test_quantized_modules_expose_weight_quantizer():
    lin = torch.nn.Linear(128, 16)
    q = jq.JenksQuantLinear(lin, 4, fmt="e2m1", group_size=32).to(DEV)
    assert torch.equal(q.weight_quantizer(), ops.dequantize(q.packed))
    conv = torch.nn.Conv2d(4, 8, 3)
    qc = jq.JenksQuantConv2d(conv, 4).to(DEV)
    assert qc.weight_quantizer().shape == conv.weight.shape


# ------------------------------------------------ pruned weights stay zero ----
def test_pruned_checkpoint_layers_on_the_gpu(golden_dir):
    """The reference's pruned LeNet-300-100 checkpoint, all three layers: the
    GPU packer reproduces the oracle's codes and codebooks, every pruned weight
    dequantises to exactly zero on the device, and the packed 784-300-100-10
    model reproduces the outputs of the reference's own forward."""
    import hashlib
    z = np.load(os.path.join(golden_dir, "lenet300_pruned_layers.npz"))
    h = torch.from_numpy(z["x"]).to(DEV)
    for li in range(3):
        W = z[f"W{li}"]
        pw = jq.pack_weight(torch.from_numpy(W).to(DEV), jq.QuantSpec("gf4", 0, 0))
        assert hashlib.sha256(pw.qweight.cpu().numpy().tobytes()).hexdigest() == str(z[f"codes_sha{li}"])
        assert np.array_equal(pw.codebook.cpu().numpy().view(np.uint16), z[f"codebook{li}"].view(np.uint16))
        w_hat = ops.dequantize(pw).cpu().numpy()
        assert np.all(w_hat[W == 0] == 0)
        y = ops.linear(h, pw, torch.from_numpy(z[f"b{li}"]).to(DEV))
        assert formats.rel_err(y.cpu().numpy(), z[f"y{li}"]) <= TOL
        h = torch.relu(y) if li < 2 else y


@pytest.mark.parametrize("B", [1, 2, 5, 12])
def test_sparse_grouped_matrix_on_the_gpu(golden_dir, B):
    z = np.load(os.path.join(golden_dir, "gf4_sparse_g128.npz"))
    W = z["W"]
    pw = jq.pack_weight(torch.from_numpy(W).to(DEV), jq.QuantSpec("gf4", 128, 0))
    assert np.array_equal(pw.qweight.cpu().numpy(), z["qweight"])
    assert np.array_equal(pw.codebook.cpu().numpy().view(np.uint16), z["codebook"].view(np.uint16))
    w_hat = ops.dequantize(pw).cpu().numpy()
    assert np.array_equal(w_hat, z["w_hat"]) and np.all(w_hat[W == 0] == 0)
    x = torch.from_numpy(np.tile(z["x"], (6, 1))[:B]).bfloat16()
    # unit vectors read columns of W_hat back through the GEMV: zeros come back as zeros (batch 1-2: pair-table
    # CUDA-core kernel, 5: 16-bit-lookup MMA loop, 12: tensor-memory kernel)
    e = torch.zeros(B, 512)
    cols = [3 + 37 * b for b in range(B)]
    for b, c in enumerate(cols):
        e[b, c] = 1.0
    y = ops.linear(e.to(DEV), pw, out_dtype=torch.float32).cpu().numpy()
    for b, c in enumerate(cols):
        assert np.array_equal(y[b], z["w_hat"][:, c])
    _check_gemv(pw.to("cpu"), x)


# ---------------------------------------------------------------- grouped ----
@pytest.mark.parametrize("fmt,g,had,B", [("gf4", 128, 128, 1), ("e2m1", 32, 0, 2), ("gf4", 128, 128, 4),
                                         ("e2m1", 32, 128, 8), ("e2m1", 32, 0, 13), ("gf4", 128, 0, 11)])
def test_grouped_launch_equals_single_launches(fmt, g, had, B):
    """Also batches above 8: one grouped launch per sub-batch of at most 8 rows."""
    shapes = [(512, 1024), (96, 2048), (1000, 256), (3, 4096), (777, 1024)]
    pws = [jq.pack_weight(_weights(n, k, n + k), jq.QuantSpec(fmt, g, had)).to(DEV) for n, k in shapes]
    grp = ops.GroupedGemv(pws, B, torch.bfloat16)
    gen = torch.Generator("cpu").manual_seed(9)
    for x in grp.xs:
        x.copy_(torch.randn(x.shape, generator=gen).bfloat16())
    for y in grp.ys:
        y.fill_(float("nan"))
    grp.run()
    torch.cuda.synchronize()
    for pw, x, y in zip(pws, grp.xs, grp.ys):
        single = ops.linear(x, pw)
        # a group runs in one kernel family; a single call picks the family by its own shape.  Where the
        # two coincide the results are identical, otherwise they differ by fp32 summation order only
        # (one bf16 rounding step at most)
        same_family = ops.ta_eligible(pw.spec.fmt_id, pw.K, pw.spec.group_size, B) == bool(grp._ta)
        if same_family:
            assert torch.equal(y, single)
        else:
            assert (y.float() - single.float()).abs().max().item() <= 2.0 ** -7 * single.float().abs().max().item()


@pytest.mark.parametrize("B,had", [(4, 0), (8, 128), (5, 0)])
def test_grouped_launch_tiles_k_when_batch_times_k_exceeds_shared_memory(B, had):
    """B x 28672 fp16 activations do not fit beside the ring: the kernel walks K in tiles and keeps fp32
    partial sums per row in shared memory (other matrices of the same launch run untiled)."""
    shapes = [(200, 28672), (48, 8192), (33, 256), (16, 28672)]
    pws = [jq.pack_weight(_weights(n, k, n + k), jq.QuantSpec("e2m1", 32, had)).to(DEV) for n, k in shapes]
    gen = torch.Generator("cpu").manual_seed(B)
    biases = [torch.randn(n, generator=gen).to(DEV) for n, _ in shapes]
    grp = ops.GroupedGemv(pws, B, torch.float32, biases=biases)
    for x in grp.xs:
        x.copy_(torch.randn(x.shape, generator=gen))
    for y in grp.ys:
        y.fill_(float("nan"))
    grp.run()
    torch.cuda.synchronize()
    assert grp.launches_per_run == 1
    for pw, x, y, b in zip(pws, grp.xs, grp.ys, biases):
        ref = ops.linear(x, pw, b)     # single launches (split-K through a workspace for the long rows)
        assert formats.rel_err(y.cpu().numpy(), ref.cpu().numpy()) <= 2e-6


@pytest.mark.parametrize("fmt,g,had,B,kmin", [("gf4", 128, 128, 1, 256), ("e2m1", 32, 0, 1, 256), ("e2m1", 32, 128, 4, 256),
                                              ("e2m1", 32, 0, 7, 256), ("gf4", 128, 128, 5, 256),
                                              ("gf4", 128, 128, 1, 512), ("gf4", 128, 128, 5, 512),
                                              ("gf4", 128, 0, 16, 512), ("e2m1", 32, 0, 16, 512), ("e2m1", 32, 128, 40, 512)])
def test_grouped_row_shards_and_peer_copies_on_one_gpu(fmt, g, had, B, kmin):
    """Two row shards of each matrix run as two grouped launches into full-width outputs; the second
    launch also writes every result into a second buffer through the peer-copy path (here a local
    buffer stands in for a peer GPU's).  Both must equal the unsharded result bit for bit.  With a
    K = 256 matrix in the set the row loops serve the group, with K >= 512 the TMA-fed kernels."""
    shapes = [(512, 1024), (96, 2048), (1000, kmin)]
    spec = jq.QuantSpec(fmt, g, had)
    full = [jq.pack_weight(_weights(n, k, n + k), spec) for n, k in shapes]
    gen = torch.Generator("cpu").manual_seed(4)
    xs = [torch.randn(B, k, generator=gen).bfloat16() for _, k in shapes]
    ref = [ops.linear(x.to(DEV), pw.to(DEV)) for x, pw in zip(xs, full)]
    halves = []
    for rank in range(2):
        shards = [pw.rows(rank * pw.N // 2, (rank + 1) * pw.N // 2).to(DEV) for pw in full]
        grp = ops.GroupedGemv(shards, B, torch.bfloat16, full_rows=[pw.N for pw in full],
                              row_offsets=[rank * pw.N // 2 for pw in full])
        for gx, x in zip(grp.xs, xs):
            gx.copy_(x)
        halves.append(grp)
    mirror = torch.zeros_like(halves[0].y_arena)
    for rank, grp in enumerate(halves):
        # copy 0 = this group's own arena, copy 1 = rank 0's arena (or the mirror when that is the same buffer)
        target = mirror if rank == 0 else halves[0].y_arena
        grp._peer_delta = np.array([0, target.data_ptr() - grp.y_arena.data_ptr()], dtype=np.int64)
        grp.run()
        assert bool(grp._ta) == (kmin >= 512) and grp.status() == 0
    torch.cuda.synchronize()
    for i, r in enumerate(ref):
        assert torch.equal(halves[0].ys[i], r)                      # own half + the half pushed by "rank 1"
        lo = full[i].N // 2
        assert torch.equal(halves[1].ys[i][:, lo:], r[:, lo:])
    esz = 2
    for i, (o, pw) in enumerate(zip(halves[0].y_offsets, full)):
        got = mirror[o:o + B * pw.N * esz].view(torch.bfloat16).view(B, pw.N)[:, : pw.N // 2]
        assert torch.equal(got, ref[i][:, : pw.N // 2])             # rank 0's half also landed in the mirror


# ----------------------------------------------------------------- conv2d ----
@pytest.mark.parametrize("fmt,g,cin,cout,k,stride,pad", [("gf4", 0, 3, 8, 3, 1, 1), ("e2m1", 32, 32, 16, 3, 2, 1),
                                                          ("e2m1", 32, 64, 24, 2, 1, 0), ("gf4", 128, 16, 12, 1, 1, 0)])
def test_quant_conv2d_matches_conv_on_dequantized_weight(fmt, g, cin, cout, k, stride, pad):
    torch.manual_seed(cin + cout)
    conv = torch.nn.Conv2d(cin, cout, k, stride=stride, padding=pad)
    q = jq.JenksQuantConv2d(conv, 4, fmt=fmt, group_size=g).to(DEV)
    x = torch.randn(2, cin, 9, 11).to(DEV)
    y = q(x)
    w_hat = q.dequantized_weight()
    ref = torch.nn.functional.conv2d(x.double(), w_hat.double(), q.bias.double(), stride=stride, padding=pad).float()
    assert y.shape == ref.shape
    assert formats.rel_err(y.cpu().numpy(), ref.cpu().numpy()) <= TOL
    q.commit()
    assert q.hard_quant and torch.equal(q(x), y)


def test_packed_checkpoint_model_runs_like_quantize_module():
    from if_i_could_turn_back_time_b200 import checkpoint
    torch.manual_seed(1)
    model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(784, 300), torch.nn.ReLU(), torch.nn.Linear(300, 10))
    spec = jq.QuantSpec("gf4", 0, 0)
    packed = checkpoint.pack_state_dict(model.state_dict(), spec)
    m1 = checkpoint.load_packed_into(torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(784, 300), torch.nn.ReLU(),
                                                         torch.nn.Linear(300, 10)), packed).to(DEV)
    m2 = jq.quantize_module(model, 4, fmt="gf4", group_size=0).to(DEV)
    x = torch.rand(3, 1, 28, 28, device=DEV)
    assert torch.equal(m1(x), m2(x))


# ------------------------------------------------------------ GPU packer ----
@pytest.mark.parametrize("N,K,g,had", [(64, 256, 32, 0), (33, 4096, 32, 128), (17, 1024, 128, 0), (5, 2048, 1024, 128)])
def test_e2m1_gpu_packer_is_bit_identical_to_host_packer(N, K, g, had):
    W = _weights(N, K, N * 3 + K)
    W[0, :g] = 0
    W[1, :32] = torch.tensor([6, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -5.0, -6] + [0] * 20) * 0.01
    if not had:
        W[2, :32] = torch.linspace(-5e5, 5e5, 32)      # absmax / 6 beyond fp16: clamped scale, saturated codes
    spec = jq.QuantSpec("e2m1", g, had)
    host = jq.pack_weight(W, spec)
    dev = jq.pack_weight(W.to(DEV), spec)
    assert dev.qweight.is_cuda
    assert torch.equal(dev.qweight.cpu(), host.qweight)
    assert torch.equal(dev.scales.cpu().view(torch.int16), host.scales.view(torch.int16))


@pytest.mark.parametrize("N,K,g,had", [(24, 1024, 128, 0), (9, 4096, 128, 128), (5, 784, 0, 0), (7, 300, 0, 0),
                                        (4, 11008, 128, 128), (3, 100, 0, 0)])
def test_gf4_gpu_packer_is_bit_identical_to_host_packer(N, K, g, had):
    W = _weights(N, K, N * 5 + K)
    spec = jq.QuantSpec("gf4", g, had)
    host = jq.pack_weight(W, spec)
    dev = jq.pack_weight(W.to(DEV), spec)
    assert torch.equal(dev.codebook.cpu().view(torch.int16), host.codebook.view(torch.int16))
    assert torch.equal(dev.qweight.cpu(), host.qweight)
    if g:
        assert torch.equal(dev.scales.cpu().view(torch.int16), host.scales.view(torch.int16))


def test_gf4_gpu_packer_ties_duplicates_and_sparse_rows():
    g = torch.Generator("cpu").manual_seed(11)
    cases = [torch.randint(-5, 6, (16, 256), generator=g).float(),
             torch.round(torch.randn(16, 512, generator=g) * 8) / 8, torch.zeros(3, 64)]
    sparse = torch.randn(10, 300, generator=g) * 0.1
    sparse[torch.rand(10, 300, generator=g) < 0.95] = 0
    cases.append(sparse)
    for W in cases:
        spec = jq.QuantSpec("gf4", 0, 0)
        host, dev = jq.pack_weight(W, spec), jq.pack_weight(W.to(DEV), spec)
        assert torch.equal(dev.codebook.cpu().view(torch.int16), host.codebook.view(torch.int16))
        assert torch.equal(dev.qweight.cpu(), host.qweight)


# ------------------------------------------------------ two-class Jenks ----
@pytest.mark.parametrize("n", [1, 2, 7, 300, 2049, 235200])
def test_two_class_jenks_break_matches_reference_form(n):
    from if_i_could_turn_back_time_b200 import prune
    from oracle import jenks as ojenks
    g = torch.Generator("cpu").manual_seed(n)
    v = torch.rand(n, generator=g) ** 3          # skewed scores, like |w * grad|
    sv = v.sort().values
    brk, vmin, gvf, var = prune.jenks2_break(sv.to(DEV), return_var=True)
    v64 = sv.double().numpy()
    if n <= 2049:   # the reference form is O(n^2): only small n
        assert brk == ojenks.two_class_break_reference_form(v64)
    # prefix-sum form in numpy float64 for every n
    s1 = np.concatenate([[0.0], np.cumsum(v64)]); s2 = np.concatenate([[0.0], np.cumsum(v64 * v64)])
    i = np.arange(n, dtype=np.float64)
    lo = np.where(i > 0, s2[:-1] - s1[:-1] ** 2 / np.maximum(i, 1), 0.0)
    hi = (s2[-1] - s2[:-1]) - (s1[-1] - s1[:-1]) ** 2 / (n - i)
    want = lo + hi
    got = var.cpu().numpy()
    assert np.allclose(got, want, rtol=1e-9, atol=1e-9 * max(1.0, abs(want).max()))
    assert abs(want[brk] - want.min()) <= 1e-9 * max(1.0, abs(want).max())
    ssd = ((v64 - v64.mean()) ** 2).sum()
    assert abs(gvf - (ssd - want.min()) / (ssd + 1e-8)) < 1e-9


def test_linear_mask_like_reference():
    from if_i_could_turn_back_time_b200 import prune
    g = torch.Generator("cpu").manual_seed(0)
    scores = torch.cat([torch.rand(900, generator=g) * 0.01, 1.0 + torch.rand(100, generator=g)])[torch.randperm(1000, generator=g)]
    mask, gvf = prune.linear_mask(scores.reshape(25, 40).to(DEV))
    assert mask.shape == (25, 40) and int(mask.sum().item()) == 100      # the upper cluster is kept
    assert torch.equal(mask.reshape(-1).bool().cpu(), scores > 0.5) and gvf > 0.95


# ------------------------------------------------- full-size property tests ----
def test_full_size_4096_e2m1_and_row_permutation():
    g = torch.Generator("cpu").manual_seed(1)
    W = (torch.randn(4096, 4096, generator=g) * 0.02).bfloat16().float()
    pw = jq.pack_weight(W, jq.QuantSpec("e2m1", 32, 0))
    x = torch.randn(1, 4096, generator=g).bfloat16()
    _check_gemv(pw, x)
    perm = torch.randperm(4096, generator=g)
    pwp = jq.PackedWeight(pw.spec, pw.N, pw.K, pw.qweight[perm], pw.scales[perm], None).to(DEV)
    y = ops.linear(x.to(DEV), pw.to(DEV), out_dtype=torch.float32)
    yp = ops.linear(x.to(DEV), pwp, out_dtype=torch.float32)
    assert torch.equal(yp[0], y[0][perm.to(DEV)])  # rows are independent: bit-exact


def test_full_size_11008_gf4_hadamard():
    g = torch.Generator("cpu").manual_seed(2)
    W = torch.randn(11008, 4096, generator=g) * 0.02
    W[torch.rand(11008, 4096, generator=g) < 0.001] *= 10
    pw = jq.pack_weight(W, jq.QuantSpec("gf4", 128, 128))
    z = torch.randn(5, 1, 4096, generator=g)
    x = z[0] / torch.sqrt((z[1:] ** 2).mean(dim=0))
    x[:, torch.randperm(4096, generator=g)[:8]] *= 50
    _check_gemv(pw, x.bfloat16())
    got = ops.dequantize(pw.to(DEV)).cpu().numpy()
    assert np.array_equal(got, _oracle_dequant(pw))
