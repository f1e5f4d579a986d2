"""Host-side mirror of the reference's QuantLinear / quantize_module surface
(no GPU: nothing here launches a kernel)."""
import inspect

import pytest
import torch
import torch.nn as nn

import if_i_could_turn_back_time_b200 as jq


def test_constructor_signature_matches_reference():
    params = list(inspect.signature(jq.JenksQuantLinear.__init__).parameters.values())
    assert [p.name for p in params[:4]] == ["self", "linear_module", "bitwidth", "mask"]
    assert params[2].default == 4 and params[3].default is None
    assert all(p.kind is inspect.Parameter.KEYWORD_ONLY for p in params[4:])


def test_attributes_and_commit():
    lin = nn.Linear(256, 24)
    q = jq.JenksQuantLinear(lin, 4, fmt="e2m1", group_size=32)
    assert isinstance(q, nn.Linear) and q.in_features == 256 and q.out_features == 24
    assert q.hard_quant is False and not q.weight.requires_grad
    assert torch.equal(q.weight.data, lin.weight.data) and torch.equal(q.bias.data, lin.bias.data)
    assert torch.equal(q.mask, torch.ones_like(lin.weight))
    q.commit()
    assert q.hard_quant is True and q._parameters["weight"] is None
    sd = q.state_dict()
    assert {"qweight", "scales", "bias", "mask"} <= set(sd) and "weight" not in sd
    assert sd["qweight"].dtype == torch.uint8 and sd["qweight"].shape == (24, 128)


def test_bitwidth_other_than_4_is_rejected():
    with pytest.raises(ValueError):
        jq.JenksQuantLinear(nn.Linear(64, 8), 8)


def test_quantize_module_swaps_linears_and_keeps_sparsity_mask():
    model = nn.Sequential(nn.Flatten(), nn.Linear(784, 300), nn.ReLU(), nn.Linear(300, 100), nn.ReLU(),
                          nn.Linear(100, 10))
    with torch.no_grad():
        model[1].weight[:, ::2] = 0
    qm = jq.quantize_module(model, 4, fmt="gf4", group_size=0)
    assert isinstance(qm[1], jq.JenksQuantLinear) and isinstance(qm[3], jq.JenksQuantLinear)
    assert isinstance(model[1], nn.Linear) and not isinstance(model[1], jq.JenksQuantLinear)  # deep copy
    assert torch.equal(qm[1].mask, (model[1].weight != 0).float())
    leaf = jq.quantize_module(nn.Linear(128, 4), 4, fmt="e2m1", group_size=32)
    assert isinstance(leaf, jq.JenksQuantLinear)


def test_forward_without_cuda_fails_loudly():
    q = jq.JenksQuantLinear(nn.Linear(64, 8), 4, fmt="e2m1", group_size=32)
    with pytest.raises(RuntimeError, match="CUDA"):
        q(torch.randn(2, 64))


def test_spec_validation():
    with pytest.raises(ValueError):
        jq.QuantSpec("e2m1", 0, 0)
    with pytest.raises(ValueError):
        jq.QuantSpec("gf4", 48, 0)
    with pytest.raises(ValueError):
        jq.QuantSpec("gf4", 128, 64)
    assert jq.algorithmic_bytes(jq.QuantSpec("e2m1", 32, 0), 4096, 4096, 1, 2, 2) == 9453568
    assert jq.algorithmic_bytes(jq.QuantSpec("gf4", 128, 128), 11008, 4096, 1, 2, 2) == 23631360


def test_status_helpers_without_any_workspace():
    """No GPU work has run: nothing to read, nothing raised; checked mode is a plain switch."""
    from if_i_could_turn_back_time_b200 import ops
    ops.set_checked(True)
    assert ops._checked is True
    ops.set_checked(False)
    assert ops._checked is False


def test_scratch_buffers_are_per_thread():
    """Calls from different host threads never share a workspace: the cache lives in thread-local storage."""
    import threading
    from if_i_could_turn_back_time_b200 import ops
    mine = ops._ws_cache()
    mine["probe"] = 1
    seen = {}

    def other():
        seen["cache"] = ops._ws_cache()
        seen["empty"] = "probe" not in seen["cache"]

    t = threading.Thread(target=other)
    t.start()
    t.join()
    del mine["probe"]
    assert seen["empty"] and seen["cache"] is not mine


def test_grouped_plan_partitions_the_row_space_evenly():
    """jq_grouped_plan is host-only: its partition of the concatenated row-group space into one contiguous range
    per CTA can be checked without a GPU (fake, aligned device addresses; nothing is dereferenced).  Layout of the
    plan: 8 header ints [magic, n, grid, largest K, rows per group, batch, format, ...], then the first row group
    of every problem (n + 1 ints) and of every CTA (grid + 1 ints)."""
    import ctypes
    import numpy as np
    from if_i_could_turn_back_time_b200 import _lib
    lib = _lib.load()
    shapes = [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)]
    n = len(shapes) * 4
    arr = (_lib.jq_problem * n)()
    for i in range(n):
        N, K = shapes[i % len(shapes)]
        arr[i].qweight = 0x10000000 + i * 0x4000000
        arr[i].scales = 0x20000000 + i * 0x400000
        arr[i].x = 0x30000000
        arr[i].y = 0x40000000
        arr[i].N, arr[i].K, arr[i].g, arr[i].had_block = N, K, 32, 0
    nbytes = lib.jq_grouped_plan_bytes(n)
    plan = np.zeros((nbytes + 3) // 4, dtype=np.int32)
    st = lib.jq_grouped_plan(_lib.JQ_FMT_E2M1, ctypes.byref(arr), n, 1, plan.ctypes.data, plan.nbytes)
    assert st == 0, _lib.strerror(st)
    grid, rows_per_group = int(plan[2]), int(plan[4])
    assert int(plan[1]) == n and grid > 0 and rows_per_group > 0
    rg_start = plan[8:8 + n + 1]
    cta_first = plan[8 + n + 1:8 + n + 1 + grid + 1]
    groups = [(-(-shapes[i % len(shapes)][0] // rows_per_group)) for i in range(n)]
    assert list(np.diff(rg_start)) == groups
    assert cta_first[0] == 0 and cta_first[-1] == rg_start[-1] and np.all(np.diff(cta_first) >= 0)
    # cost of every CTA's range in row-group x K units: within two row groups of the mean
    k_of = np.repeat([shapes[i % len(shapes)][1] for i in range(n)], groups)
    cost = np.array([k_of[a:b].sum() for a, b in zip(cta_first[:-1], cta_first[1:])], dtype=np.float64)
    assert abs(cost - cost.mean()).max() <= 2 * 11008
    # a misaligned weight pointer is refused before anything else happens
    arr[3].qweight += 8
    st = lib.jq_grouped_plan(_lib.JQ_FMT_E2M1, ctypes.byref(arr), n, 1, plan.ctypes.data, plan.nbytes)
    assert st != 0 and "align" in _lib.strerror(st)
