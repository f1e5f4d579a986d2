"""Generate the committed golden vectors under tests/golden/.

Run once on a machine that has the reference checkout:
    python tests/golden/make_golden.py <path to the reference checkout>
The reference has no packed format, so the *format* side of every vector
comes from the CPU oracle (oracle/formats.py, oracle/jenks.py).  The
*operator* side is the reference's own code: its ``QuantLinear`` class
(Python_Jenks_Test/Jenks_Tests/Quantization_Experiments/layers.py:11-45) is
loaded by file path, put in hard-quant mode with its weight overwritten by
the oracle-dequantized matrix, and its ``forward`` (``F.linear`` in fp32,
layers.py:34-35) produces the expected outputs.  One vector uses rows of the
reference's pruned LeNet-300-100 checkpoint
(Python_Jenks_Test/Jenks_Tests/Best_Results_HPO/LeNet300/best_2025-12-09_18-58-19_MNIST_LeNet300.pth),
which exercises the "fewer than 16 distinct values" path.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import formats, jenks  # noqa: E402


def load_reference_quantlinear(ref_root: str):
    path = os.path.join(ref_root, "Python_Jenks_Test", "Jenks_Tests", "Quantization_Experiments", "layers.py")
    spec = importlib.util.spec_from_file_location("ref_layers", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.QuantLinear


def load_reference_brecq(ref_root: str):
    """``UniformAffineQuantizer``, ``AdaRoundQuantizer`` and ``replace_forward`` of the reference's brecq.py
    (Quantization_Experiments/brecq.py:13-92, 305-331).  The file's own imports need packages that are not
    installed (and sibling modules on sys.path), so only these three definitions are compiled, from the
    reference's source text, in a namespace that has torch."""
    import ast
    import contextlib
    import io
    path = os.path.join(ref_root, "Python_Jenks_Test", "Jenks_Tests", "Quantization_Experiments", "brecq.py")
    tree = ast.parse(open(path).read())
    want = {"UniformAffineQuantizer", "AdaRoundQuantizer", "replace_forward"}
    body = [n for n in tree.body if isinstance(n, (ast.ClassDef, ast.FunctionDef)) and n.name in want]
    ns = {"torch": torch, "nn": torch.nn, "F": torch.nn.functional}
    exec(compile(ast.Module(body=body, type_ignores=[]), path, "exec"), ns)
    ns["_quiet"] = lambda: contextlib.redirect_stdout(io.StringIO())   # the classes print while they work
    return ns


def ref_forward(QuantLinear, w_hat: np.ndarray, bias, x: np.ndarray) -> np.ndarray:
    N, K = w_hat.shape
    lin = torch.nn.Linear(K, N, bias=bias is not None)
    q = QuantLinear(lin, bitwidth=4)
    with torch.no_grad():
        q.weight.data.copy_(torch.from_numpy(w_hat))
        if bias is not None:
            q.bias.data.copy_(torch.from_numpy(bias))
    q.hard_quant = True
    with torch.no_grad():
        return q(torch.from_numpy(x)).numpy()


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).bfloat16().float().numpy()


def main(ref_root: str) -> None:
    QL = load_reference_quantlinear(ref_root)
    torch.set_num_threads(1)

    # ---- KAT: every byte -> two E2M1 values --------------------------------
    allbytes = np.arange(256, dtype=np.uint8).reshape(1, 256)          # one row of 512 codes
    codes = formats.unpack_nibbles(allbytes, 512)
    vals = formats.dequant_e2m1(codes, np.ones((1, 16), dtype=np.float16), 32)
    np.savez(os.path.join(HERE, "kat_e2m1_bytes.npz"), qweight=allbytes, values=vals)

    # ---- KAT: Hadamard of unit vectors = rows of H/sqrt(128) ---------------
    eye = np.eye(128, dtype=np.float32)
    np.savez(os.path.join(HERE, "kat_fwht128.npz"), rows=formats.fwht_block(eye, 128))

    # ---- config-1 MLP 784-300-100-10, GF4 without groups -------------------
    g = torch.Generator("cpu").manual_seed(0)
    dims = [(300, 784), (100, 300), (10, 100)]
    Ws = [(torch.randn(n, k, generator=g) * k ** -0.5).numpy() for n, k in dims]
    x = torch.rand(1, 784, generator=g).numpy()
    out = {"x": x}
    h = x
    for li, W in enumerate(Ws):
        c, cb, _ = jenks.quantize_gf4(W, 0)
        w_hat = formats.dequant_gf4(c, cb, None, 0)
        y = ref_forward(QL, w_hat, None, h)
        out[f"codebook{li}"] = cb
        out[f"codes_sha{li}"] = np.array(sha(formats.pack_nibbles(c)))
        out[f"what_sha{li}"] = np.array(sha(w_hat))
        out[f"y{li}"] = y
        h = np.maximum(y, 0) if li < 2 else y
    np.savez(os.path.join(HERE, "mlp_gf4.npz"), **out)

    # ---- E2M1 g32, bf16 weights and activations, with bias -----------------
    g = torch.Generator("cpu").manual_seed(1)
    W = (torch.randn(64, 256, generator=g) * 0.02).bfloat16().float().numpy()
    xb = torch.randn(4, 256, generator=g).bfloat16().float().numpy()
    bias = torch.randn(64, generator=g).numpy()
    c, s = formats.quantize_e2m1(W, 32)
    w_hat = formats.dequant_e2m1(c, s, 32)
    np.savez(os.path.join(HERE, "e2m1_g32.npz"), W=W, x=xb, bias=bias, qweight=formats.pack_nibbles(c), scales=s,
             w_hat=w_hat, y=ref_forward(QL, w_hat, bias, xb))

    # ---- GF4 g128 + Hadamard, outlier weights, heavy-tailed activations -----
    g = torch.Generator("cpu").manual_seed(2)
    W = torch.randn(32, 512, generator=g) * 0.02
    W[torch.rand(32, 512, generator=g) < 0.001] *= 10
    W = W.numpy()
    z = torch.randn(5, 2, 512, generator=g)
    xt = z[0] / torch.sqrt((z[1:] ** 2).mean(dim=0))
    xt[:, torch.randperm(512, generator=g)[:8]] *= 50
    xt = xt.bfloat16().float().numpy()
    Wr = formats.fwht_block(W, 128)
    c, cb, s = jenks.quantize_gf4(Wr, 128)
    w_hat = formats.dequant_gf4(c, cb, s, 128)
    x_rot = formats.fwht_block(xt, 128)
    np.savez(os.path.join(HERE, "gf4_g128_had.npz"), W=W, x=xt, qweight=formats.pack_nibbles(c), scales=s,
             codebook=cb, w_hat=w_hat, x_rot=x_rot, y=ref_forward(QL, w_hat, None, x_rot))

    # ---- rows of the reference's pruned LeNet-300-100 checkpoint ------------
    ck = os.path.join(ref_root, "Python_Jenks_Test", "Jenks_Tests", "Best_Results_HPO", "LeNet300",
                      "best_2025-12-09_18-58-19_MNIST_LeNet300.pth")
    sd = torch.load(ck, map_location="cpu", weights_only=True)
    W = sd["1.weight"][:24].float().numpy()
    g = torch.Generator("cpu").manual_seed(5)
    x = torch.rand(2, 784, generator=g).numpy()
    c, cb, _ = jenks.quantize_gf4(W, 0)
    w_hat = formats.dequant_gf4(c, cb, None, 0)
    np.savez_compressed(os.path.join(HERE, "lenet300_pruned_rows.npz"), W=W, x=x, qweight=formats.pack_nibbles(c),
                        codebook=cb, y=ref_forward(QL, w_hat, None, x))

    # ---- all three layers of that checkpoint (97.8 % zeros): pruned weights must come back as exact zeros ----
    Ws = [sd[f"{i}.weight"].float().numpy() for i in (1, 3, 5)]
    bs = [sd[f"{i}.bias"].float().numpy() for i in (1, 3, 5)]
    g = torch.Generator("cpu").manual_seed(6)
    x = torch.rand(3, 784, generator=g).numpy()
    out = {"x": x}
    h = x
    for li, (W, b) in enumerate(zip(Ws, bs)):
        c, cb, _ = jenks.quantize_gf4(W, 0)
        w_hat = formats.dequant_gf4(c, cb, None, 0)
        assert np.all(w_hat[W == 0] == 0), "a pruned weight did not stay zero"
        y = ref_forward(QL, w_hat, b, h)
        out[f"W{li}"], out[f"b{li}"], out[f"codebook{li}"], out[f"y{li}"] = W, b, cb, y
        out[f"codes_sha{li}"] = np.array(sha(formats.pack_nibbles(c)))
        h = np.maximum(y, 0) if li < 2 else y
    np.savez_compressed(os.path.join(HERE, "lenet300_pruned_layers.npz"), **out)

    # ---- a half-pruned matrix with group scales: zeros survive the group normalisation too -------------------
    g = torch.Generator("cpu").manual_seed(7)
    W = torch.randn(16, 512, generator=g) * 0.02
    W[torch.rand(16, 512, generator=g) < 0.5] = 0.0
    W[3] = 0.0                                   # an all-zero row (scale guard, one distinct value)
    W[5, :128] = 0.0                             # an all-zero group
    W = W.numpy()
    x = torch.randn(2, 512, generator=g).bfloat16().float().numpy()
    c, cb, s = jenks.quantize_gf4(W, 128)
    w_hat = formats.dequant_gf4(c, cb, s, 128)
    assert np.all(w_hat[W == 0] == 0)
    np.savez_compressed(os.path.join(HERE, "gf4_sparse_g128.npz"), W=W, x=x, qweight=formats.pack_nibbles(c), scales=s,
                        codebook=cb, w_hat=w_hat, y=ref_forward(QL, w_hat, None, x))

    # ---- the BRECQ boundary: a Linear whose forward the reference's replace_forward has swapped -----------------
    bq = load_reference_brecq(ref_root)
    g = torch.Generator("cpu").manual_seed(8)
    lin = torch.nn.Linear(256, 48)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(48, 256, generator=g) * 0.05)
        lin.weight[torch.rand(48, 256, generator=g) < 0.3] = 0.0       # pruned entries: AdaRound keeps them at zero
        lin.bias.copy_(torch.randn(48, generator=g) * 0.1)
    x = torch.randn(5, 256, generator=g)
    with bq["_quiet"](), torch.no_grad():
        quantizer = bq["AdaRoundQuantizer"](lin.weight.data, bq["UniformAffineQuantizer"](bitwidth=4))
        frac = lin.weight.data / quantizer.quantizer.delta - quantizer.W_floor
        quantizer.alpha.copy_(torch.where(frac > 0.5, torch.tensor(20.0), torch.tensor(-20.0)))   # converged: hard rounding
        lin.weight_quantizer = quantizer
        bq["replace_forward"](lin)
        y = lin(x)
        w_q = quantizer()
    np.savez_compressed(os.path.join(HERE, "brecq_replace_forward.npz"), W=lin.weight.data.numpy(), W_q=w_q.numpy(),
                        bias=lin.bias.data.numpy(), x=x.numpy(), y=y.numpy())
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
