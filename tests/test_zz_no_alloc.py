"""The allocation-free entry point, jq_gemv_noalloc.

Some callers of this library may not allocate GPU memory at all: code that
runs inside an allocator callback (calling cudaMalloc there can deadlock the
allocator), a real-time loop whose memory budget was fixed when it started,
or a host that passes only the layer's tensors and has no workspace to lend.
For them the split-K partial sums live in an array built into the library.
The test calls that entry straight through the C ABI, twice in a row with
different inputs (the array keeps the first call's contents), and compares
each result with the ordinary entry point that uses a caller workspace (the
two run the same kernels in the same order, so they must agree bit for bit)
and with the CPU oracle.
It is collected last so that a run stopping at the first failure has already
run everything else, and it needs nothing from the other tests.
"""
import ctypes

import numpy as np
import pytest
import torch

import if_i_could_turn_back_time_b200 as jq
from if_i_could_turn_back_time_b200 import _lib
from oracle import formats

pytestmark = pytest.mark.gpu
TOL = 1e-3  # the GEMV gate used by the other GPU tests: max|y - y_ref| / max|y_ref|
DEV = "cuda:0"


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("fmt,g", [("e2m1", 32), ("gf4", 128)])
def test_noalloc_matches_workspace_entry_twice(fmt, g):
    lib = _lib.load()
    N, K, B = 96, 28672, 8           # B x K does not fit in shared memory: the split-K path, which needs scratch
    ws_bytes = lib.jq_workspace_bytes(0, N, K, B)
    assert 0 < ws_bytes <= (8 << 20)
    gen = torch.Generator("cpu").manual_seed(11)
    W = torch.randn(N, K, generator=gen) * 0.02
    pw = jq.pack_weight(W, jq.QuantSpec(fmt, g, 128)).to(DEV)
    bias = torch.randn(N, generator=gen).to(DEV)
    fmt_id = _lib.JQ_FMT_E2M1 if fmt == "e2m1" else _lib.JQ_FMT_GF4
    codes = formats.unpack_nibbles(pw.qweight.cpu().numpy(), K)
    w_hat = (formats.dequant_e2m1(codes, pw.scales.cpu().numpy(), g) if fmt == "e2m1"
             else formats.dequant_gf4(codes, pw.codebook.cpu().numpy(), pw.scales.cpu().numpy(), g))
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        x = (torch.randn(B, K, generator=gen) * (1.0 + 3.0 * call)).bfloat16().to(DEV)
        y_new = torch.full((B, N), float("nan"), dtype=torch.float32, device=DEV)
        y_old = torch.full((B, N), float("nan"), dtype=torch.float32, device=DEV)
        st = lib.jq_gemv_noalloc(fmt_id, _p(pw.qweight), _p(pw.scales), _p(pw.codebook), _p(x), _p(bias), _p(y_new),
                                 N, K, B, g, 128, _lib.JQ_BF16, _lib.JQ_F32, stream)
        assert st == 0, _lib.strerror(st)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
        if fmt == "e2m1":
            st = lib.jq_gemv_e2m1(_p(pw.qweight), _p(pw.scales), _p(x), _p(bias), _p(y_old), N, K, B, g, 128,
                                  _lib.JQ_BF16, _lib.JQ_F32, _p(ws), ws_bytes, stream)
        else:
            st = lib.jq_gemv_gf4(_p(pw.qweight), _p(pw.scales), _p(pw.codebook), _p(x), _p(bias), _p(y_old), N, K, B,
                                 g, 128, _lib.JQ_BF16, _lib.JQ_F32, _p(ws), ws_bytes, stream)
        assert st == 0, _lib.strerror(st)
        torch.cuda.synchronize()
        a, b = y_new.cpu().numpy(), y_old.cpu().numpy()
        assert np.isfinite(a).all()
        assert torch.equal(y_new, y_old), f"call {call}: {formats.rel_err(a, b):.3e}"
        ref = formats.linear_ref(x.float().cpu().numpy(), w_hat, bias.cpu().numpy(), had_block=128)
        assert formats.rel_err(a, ref) <= TOL, f"call {call} vs oracle: {formats.rel_err(a, ref):.3e}"


def test_noalloc_rejects_problems_beyond_the_builtin_scratch():
    lib = _lib.load()
    x = torch.zeros(8, dtype=torch.uint8, device=DEV)  # pointers only pass validation; nothing is launched
    p = ctypes.c_void_p(x.data_ptr())
    st = lib.jq_gemv_noalloc(_lib.JQ_FMT_E2M1, p, p, None, p, None, p, 1 << 20, 28672, 8, 32, 0, _lib.JQ_BF16,
                             _lib.JQ_BF16, None)
    assert st == -9 and "scratch" in _lib.strerror(st)
