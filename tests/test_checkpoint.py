"""Packed checkpoint format: float state_dict -> packed dict -> file -> model (no GPU)."""
import io

import numpy as np
import torch
import torch.nn as nn

import if_i_could_turn_back_time_b200 as jq
from if_i_could_turn_back_time_b200 import checkpoint
from oracle import formats


def _lenet():
    return nn.Sequential(nn.Flatten(), nn.Linear(784, 300), nn.ReLU(), nn.Linear(300, 100), nn.ReLU(), nn.Linear(100, 10))


def test_pack_save_load_roundtrip():
    torch.manual_seed(0)
    model = _lenet()
    with torch.no_grad():
        model[1].weight[model[1].weight.abs() < 0.03] = 0      # a pruned layer, like the reference's checkpoints
    sd = model.state_dict()                                     # keys 1.weight, 1.bias, 3.weight, ... as in the reference
    packed = checkpoint.pack_state_dict(sd, jq.QuantSpec("gf4", 0, 0))
    assert set(packed) == {"1.qweight", "1.codebook", "1.meta", "1.bias", "3.qweight", "3.codebook", "3.meta", "3.bias",
                           "5.qweight", "5.codebook", "5.meta", "5.bias"}
    assert packed["1.qweight"].shape == (300, 400) and packed["1.meta"].tolist() == [1, 0, 0, 300, 784]
    buf = io.BytesIO()
    torch.save(packed, buf)
    buf.seek(0)
    loaded = torch.load(buf, weights_only=True)
    new = checkpoint.load_packed_into(_lenet(), loaded)
    for idx in (1, 3, 5):
        m = new[idx]
        assert isinstance(m, jq.JenksQuantLinear) and m.hard_quant and m._parameters["weight"] is None
        assert torch.equal(m.qweight, packed[f"{idx}.qweight"]) and torch.equal(m.bias, sd[f"{idx}.bias"])
    # zeros survive quantisation exactly (sparsity of the pruned layer is preserved)
    pw = checkpoint.packed_weight_from(loaded, "1")
    codes = formats.unpack_nibbles(pw.qweight.numpy(), pw.K)
    w_hat = formats.dequant_gf4(codes, pw.codebook.numpy(), None, 0)
    zero = sd["1.weight"].numpy() == 0
    assert zero.mean() > 0.3 and np.all(w_hat[zero] == 0)
    # the packed file is ~8x smaller than the float one
    fbuf = io.BytesIO()
    torch.save(sd, fbuf)
    assert len(buf.getvalue()) < len(fbuf.getvalue()) / 6


def test_group_spec_falls_back_when_k_does_not_divide():
    sd = {"a.weight": torch.randn(8, 256), "b.weight": torch.randn(8, 100), "c.weight": torch.randn(4)}
    packed = checkpoint.pack_state_dict(sd, jq.QuantSpec("gf4", 128, 128))
    assert packed["a.meta"].tolist() == [1, 128, 128, 8, 256]
    assert packed["b.meta"].tolist() == [1, 0, 0, 8, 100] and "b.scales" not in packed
    assert torch.equal(packed["c.weight"], sd["c.weight"])
