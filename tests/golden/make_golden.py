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
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
