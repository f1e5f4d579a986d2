"""Operators over packed weights: thin, checked calls into libjq.so.

Everything here runs on the GPU through the C ABI; there is no eager or CPU
fallback.  The fused linear is also registered as ``torch.ops.jq.linear`` so
that it composes with torch's dispatcher (fake tensors, export).
"""
from __future__ import annotations

import ctypes
import threading
import warnings
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib
from .pack import PackedWeight

_DT = {torch.float32: _lib.JQ_F32, torch.float16: _lib.JQ_F16, torch.bfloat16: _lib.JQ_BF16}
MAX_GEMV_BATCH = 8


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("libjq operators run on CUDA tensors only (there is no CPU path)")


def dequantize(pw: PackedWeight) -> torch.Tensor:
    """Dense fp32 [N, K] of a packed matrix (bit-exact definition of W_hat)."""
    lib = _lib.load()
    _need_cuda(pw.qweight, pw.scales, pw.codebook)
    out = torch.empty((pw.N, pw.K), dtype=torch.float32, device=pw.qweight.device)
    with torch.cuda.device(out.device):
        if pw.spec.fmt == "e2m1":
            st = lib.jq_dequant_e2m1(_ptr(pw.qweight), _ptr(pw.scales), _ptr(out), pw.N, pw.K, pw.spec.group_size,
                                     _stream())
        else:
            st = lib.jq_dequant_gf4(_ptr(pw.qweight), _ptr(pw.scales), _ptr(pw.codebook), _ptr(out), pw.N, pw.K,
                                    pw.spec.group_size, _stream())
    _lib.check(st, "jq_dequant")
    return out


def fwht_block(x: torch.Tensor, block: int = 128) -> torch.Tensor:
    """fp32 block Hadamard rotation along the last dim."""
    lib = _lib.load()
    _need_cuda(x)
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    y = torch.empty(x2.shape, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        st = lib.jq_fwht_block(_ptr(x2), _ptr(y), x2.shape[0], x2.shape[1], block, _DT[x2.dtype], _stream())
    _lib.check(st, "jq_fwht_block")
    return y.reshape(x.shape)


_OUT = {-1: None, _lib.JQ_F32: torch.float32, _lib.JQ_F16: torch.float16, _lib.JQ_BF16: torch.bfloat16}


def ta_max_batch(fmt_id: int) -> int:
    """Rows one pass of the pair-table / tensor-memory kernels takes."""
    return 16 if fmt_id == _lib.JQ_FMT_GF4 else 64


def ta_eligible(fmt_id: int, K: int, g: int, batch: int) -> bool:
    """Problems the TMA-fed kernels take.  GF4 (group size 128 * 2^k): every
    batch -- one row (while the prepared activation fits in shared memory, K
    up to 12288) on the CUDA-core pair-table loop, the rest on the
    tensor-memory kernel, 16 rows per pass.  E2M1 g32: batches from 9 rows on
    the tensor-memory kernel, 64 rows per pass (up to 8 rows the mma.sync row
    loops are faster)."""
    if K % 256 or K < 512:
        return False
    if fmt_id == _lib.JQ_FMT_GF4:
        gq = g >> 7
        return g >= 128 and g % 128 == 0 and gq & (gq - 1) == 0 and K % g == 0 and batch >= 1
    return g == 32 and batch >= 9


def _ta_aligned(*tensors) -> bool:
    """The TMA-fed kernels read E2M1 scales in 16-byte pieces (the row loops in 2- or 4-byte pieces); a view that
    starts elsewhere is served by the row loops instead.  Packed rows and codebooks are 16-byte aligned on every
    path (the library refuses anything else)."""
    return all(t is None or t.data_ptr() % 16 == 0 for t in tensors)


_tls = threading.local()   # every host thread has its own scratch buffers: calls from different threads never share one
_checked = False


def _ws_cache() -> dict:
    d = getattr(_tls, "ws", None)
    if d is None:
        d = _tls.ws = {}
    return d


def set_checked(on: bool) -> None:
    """Checked mode: every call that runs a kernel with device-side waits (the
    pair-table and tensor-memory kernels) is followed by a read of its status
    word, which synchronises the stream, and raises if a wait gave up.  Off by
    default: the status stays in the workspace until ``check_status()``."""
    global _checked
    _checked = bool(on)


def _workspace(device, nbytes: int, kind: str = "gemv") -> torch.Tensor:
    """Grow-only scratch per (device, stream, kernel family): calls on one
    stream are ordered, so consecutive calls may share it; another stream gets
    its own.  The family with a status word at offset 0 ("ta") never shares
    a buffer with the split-K partial sums, and starts zeroed."""
    key = (device, torch.cuda.current_stream(device).cuda_stream, kind)
    cache = _ws_cache()
    t = cache.get(key)
    if t is None or t.numel() < nbytes:
        if t is not None and kind != "gemv" and check_status(raise_on_error=False):
            raise RuntimeError("a device-side wait gave up in an earlier call (status word raised)")
        t = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        cache[key] = t
    return t


def reserve_workspace(device, nbytes: int, kind: str = "ta") -> None:
    """Allocate this thread's scratch for (device, current stream, kernel family) ahead of time, e.g. before a
    CUDA-graph capture or a region that must not allocate: kind "gemv" = split-K partial sums of the row loops,
    "ta" = prepared activations and status word of the TMA-fed kernels."""
    _workspace(torch.device(device), nbytes, kind)


def check_status(raise_on_error: bool = True) -> int:
    """Read and clear the sticky status words of this device's workspaces on
    the current stream (synchronises).  A kernel whose bounded wait expired
    leaves JQ_ERR_TIMEOUT there and returns early with its outputs partly
    written; every later call keeps the word until it is read here."""
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    worst = 0
    ws = _ws_cache().get((dev, stream, "ta"))
    if ws is not None:
        worst = min(worst, lib.jq_ta_status(_ptr(ws), 1, _stream()))
    if worst and raise_on_error:
        raise _lib.JqError(worst, "device status")
    return worst


def _linear_rows_ta(x2, qweight, scales, codebook, bias, fmt_id, N, K, g, had, y):
    """Through the TMA-fed kernels, at most ta_max_batch rows per pass."""
    lib = _lib.load()
    Bt = x2.shape[0]
    MAX_TA_BATCH = ta_max_batch(fmt_id)
    prob = _lib.jq_problem()
    prob.K = K
    with _on(x2.device):
        stream = _stream()
        for b0 in range(0, Bt, MAX_TA_BATCH):
            b1 = min(Bt, b0 + MAX_TA_BATCH)
            wsb = lib.jq_ta_workspace_bytes(ctypes.byref(prob), 1, b1 - b0)
            ws = _workspace(x2.device, wsb, "ta")
            xs, ys = (x2, y) if Bt <= MAX_TA_BATCH else (x2[b0:b1], y[b0:b1])
            st = lib.jq_gemm_ta(fmt_id, _ptr(qweight), _ptr(scales), _ptr(codebook), _ptr(xs), _ptr(bias),
                                _ptr(ys), N, K, b1 - b0, g, had, _DT[x2.dtype], _DT[y.dtype], _ptr(ws), ws.numel(), stream)
            _lib.check(st, "jq_gemm_ta")
    if _checked:
        check_status()
    return y


_wsb_cache = {}


class _NoDeviceSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoDeviceSwitch()


def _on(device):
    """Device guard that costs nothing when the tensor's device is already current."""
    return _NO_SWITCH if device.index == torch.cuda.current_device() else torch.cuda.device(device)


def _linear_rows(x2, qweight, scales, codebook, bias, fmt_id, N, K, g, had, out_id=-1):
    lib = _lib.load()
    Bt = x2.shape[0]
    y = torch.empty((Bt, N), dtype=_OUT[out_id] or x2.dtype, device=x2.device)
    if ta_eligible(fmt_id, K, g, Bt) and _ta_aligned(qweight, scales, codebook):
        return _linear_rows_ta(x2, qweight, scales, codebook, bias, fmt_id, N, K, g, had, y)
    xd, yd = _DT[x2.dtype], _DT[y.dtype]
    qw_p, sc_p, cb_p, bias_p = _ptr(qweight), _ptr(scales), _ptr(codebook), _ptr(bias)
    with _on(x2.device):
        stream = _stream()
        for b0 in range(0, Bt, MAX_GEMV_BATCH):
            b1 = min(Bt, b0 + MAX_GEMV_BATCH)
            xs, ys = (x2, y) if Bt <= MAX_GEMV_BATCH else (x2[b0:b1], y[b0:b1])
            # split-K scratch (fp32 partial outputs) when the staged batch would not fit in shared memory
            key = (N, K, b1 - b0)
            wsb = _wsb_cache.get(key)
            if wsb is None:
                wsb = _wsb_cache[key] = lib.jq_workspace_bytes(0, N, K, b1 - b0)
            ws = _workspace(x2.device, wsb)[:wsb] if wsb else None

            def call(ws_t):
                nb = ws_t.numel() if ws_t is not None else 0
                if fmt_id == _lib.JQ_FMT_E2M1:
                    return lib.jq_gemv_e2m1(qw_p, sc_p, _ptr(xs), bias_p, _ptr(ys), N, K,
                                            b1 - b0, g, had, xd, yd, _ptr(ws_t), nb, stream)
                return lib.jq_gemv_gf4(qw_p, sc_p, cb_p, _ptr(xs), bias_p, _ptr(ys),
                                       N, K, b1 - b0, g, had, xd, yd, _ptr(ws_t), nb, stream)

            st = call(ws)
            if st == -6 and ws is not None:   # workspace too small for this group size: sub-batch path
                st = call(None)
            if st:
                _lib.check(st, "jq_gemv")
    return y


@torch.library.custom_op("jq::linear", mutates_args=(), device_types="cuda")
def _jq_linear(x: torch.Tensor, qweight: torch.Tensor, scales: Optional[torch.Tensor],
               codebook: Optional[torch.Tensor], bias: Optional[torch.Tensor], fmt_id: int, N: int, K: int,
               group_size: int, had_block: int, out_id: int) -> torch.Tensor:
    x2 = x.reshape(-1, K).contiguous()
    y = _linear_rows(x2, qweight, scales, codebook, bias, fmt_id, N, K, group_size, had_block, out_id)
    return y.reshape(*x.shape[:-1], N)


@_jq_linear.register_fake
def _(x, qweight, scales, codebook, bias, fmt_id, N, K, group_size, had_block, out_id):
    return x.new_empty((*x.shape[:-1], N), dtype=_OUT[out_id] or x.dtype)


def linear(x: torch.Tensor, pw: PackedWeight, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``F.linear(rotate(x), W_hat, bias)`` without materialising W_hat; any
    leading dims, last dim = K; output dtype = input dtype unless given."""
    if x.shape[-1] != pw.K:
        raise RuntimeError(f"last dim of x is {x.shape[-1]}, packed weight has K={pw.K}")
    if x.dtype not in _DT:
        raise RuntimeError(f"unsupported activation dtype {x.dtype}")
    _need_cuda(x, pw.qweight, pw.scales, pw.codebook, bias)
    if bias is not None and bias.dtype != torch.float32:
        bias = bias.float()
    out_id = -1 if out_dtype is None else _DT[out_dtype]
    if torch.compiler.is_compiling():
        # through the dispatcher so that tracing sees one opaque op with a fake implementation
        return torch.ops.jq.linear(x, pw.qweight, pw.scales, pw.codebook, bias, pw.spec.fmt_id, pw.N, pw.K,
                                   pw.spec.group_size, pw.spec.had_block, out_id)
    x2 = x.reshape(-1, pw.K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = _linear_rows(x2, pw.qweight, pw.scales, pw.codebook, bias, pw.spec.fmt_id, pw.N, pw.K, pw.spec.group_size,
                     pw.spec.had_block, out_id)
    return y.reshape(*x.shape[:-1], pw.N)


class GroupedGemv:
    """A fixed set of independent GEMVs (one decode step's matrices) run in a
    single launch.  Inputs and outputs are preallocated; ``run()`` only
    enqueues the kernel.

    Row-sharded use (one process per GPU): pass each matrix's local shard in
    ``weights``, its unsharded row count in ``full_rows`` and the shard's
    first row in ``row_offsets``; outputs are then full-width ``[batch,
    full_rows]`` buffers of which this rank fills its columns.  With
    ``group`` (a ``torch.distributed`` process group, world size <= 8) the
    output arena lives in symmetric memory and the kernel's epilogue stores
    every result into all ranks' arenas (the all-gather fused into the GEMV);
    call ``barrier()`` after ``run()`` before reading."""

    def __init__(self, weights: Sequence[PackedWeight], batch: int, x_dtype=torch.bfloat16,
                 biases: Optional[Sequence[Optional[torch.Tensor]]] = None, device=None,
                 full_rows: Optional[Sequence[int]] = None, row_offsets: Optional[Sequence[int]] = None,
                 group=None):
        lib = _lib.load()
        if not weights:
            raise ValueError("no problems")
        spec0 = weights[0].spec
        for w in weights:
            if w.spec.fmt != spec0.fmt:
                raise ValueError("a grouped launch needs one weight format")
        self.device = device or weights[0].qweight.device
        self.weights = list(weights)
        self.batch = batch
        self.x_dtype = x_dtype
        self.biases = list(biases) if biases is not None else [None] * len(weights)
        self.full_rows = list(full_rows) if full_rows is not None else [w.N for w in weights]
        self.row_offsets = list(row_offsets) if row_offsets is not None else [0] * len(weights)
        # all inputs live in one arena and all outputs in another, so a step's
        # activations move with one copy each way; every view is 256-byte aligned
        esz = torch.empty((), dtype=x_dtype).element_size()
        rnd = lambda nbytes: (nbytes + 255) // 256 * 256
        x_off, y_off, xo, yo = [], [], 0, 0
        for w, nf in zip(weights, self.full_rows):
            x_off.append(xo); xo += rnd(batch * w.K * esz)
            y_off.append(yo); yo += rnd(batch * nf * esz)
        self.x_arena = torch.zeros(xo, dtype=torch.uint8, device=self.device)
        self._symm = None
        self._peer_delta = np.zeros(1, dtype=np.int64)
        if group is not None and torch.distributed.get_world_size(group) > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.y_arena = symm_mem.empty(yo, dtype=torch.uint8, device=self.device)
            self.y_arena.zero_()
            self._symm = symm_mem.rendezvous(self.y_arena, group.group_name if hasattr(group, "group_name") else group)
            own = self.y_arena.data_ptr()
            ptrs = [int(p) for p in self._symm.buffer_ptrs]
            if len(ptrs) > 8:
                raise ValueError("at most 8 peers")
            self._peer_delta = np.array([p - own for p in ptrs], dtype=np.int64)
        else:
            self.y_arena = torch.zeros(yo, dtype=torch.uint8, device=self.device)
        self.x_offsets, self.y_offsets = x_off, y_off
        self.xs: List[torch.Tensor] = [
            self.x_arena[o:o + batch * w.K * esz].view(x_dtype).view(batch, w.K) for o, w in zip(x_off, weights)]
        self.ys: List[torch.Tensor] = [
            self.y_arena[o:o + batch * nf * esz].view(x_dtype).view(batch, nf) for o, nf in zip(y_off, self.full_rows)]
        n = len(weights)
        arr = (_lib.jq_problem * n)()
        for i, w in enumerate(weights):
            arr[i].qweight = w.qweight.data_ptr()
            arr[i].scales = w.scales.data_ptr() if w.scales is not None else None
            arr[i].codebook = w.codebook.data_ptr() if w.codebook is not None else None
            arr[i].x = self.xs[i].data_ptr()
            arr[i].bias = self.biases[i].data_ptr() if self.biases[i] is not None else None
            arr[i].y = self.ys[i].data_ptr() + self.row_offsets[i] * esz
            arr[i].N, arr[i].K, arr[i].g, arr[i].had_block = w.N, w.K, w.spec.group_size, w.spec.had_block
            arr[i].ldy = self.full_rows[i]
        self._problems_host = arr
        self._per_problem = False
        self._subs = []
        self._ta = []
        use_ta = all(ta_eligible(w.spec.fmt_id, w.K, w.spec.group_size, batch)
                     and _ta_aligned(w.qweight, w.scales, w.codebook) for w in weights)
        if use_ta:
            MAX_TA_BATCH = ta_max_batch(spec0.fmt_id)
            # through the TMA-fed kernels: one plan (and workspace) per sub-batch of at most 16 (GF4) or 64 (E2M1)
            # rows; a run is one activation-preparation launch plus one persistent launch per sub-batch
            with torch.cuda.device(self.device):
                for b0 in range(0, batch, MAX_TA_BATCH):
                    nb = min(MAX_TA_BATCH, batch - b0)
                    sub = (_lib.jq_problem * n)()
                    ctypes.memmove(sub, arr, ctypes.sizeof(arr))
                    for i, (w, nf) in enumerate(zip(weights, self.full_rows)):
                        sub[i].x = arr[i].x + b0 * w.K * esz
                        sub[i].y = arr[i].y + b0 * nf * esz
                    wsb = lib.jq_ta_workspace_bytes(ctypes.byref(sub), n, nb)
                    ws = torch.zeros(wsb, dtype=torch.uint8, device=self.device)
                    plan_host = np.zeros((lib.jq_ta_plan_bytes(n) + 3) // 4, dtype=np.int32)
                    _lib.check(lib.jq_ta_plan(spec0.fmt_id, ctypes.byref(sub), n, nb, _ptr(ws), wsb,
                                              plan_host.ctypes.data, plan_host.nbytes), "jq_ta_plan")
                    self._ta.append((plan_host, torch.from_numpy(plan_host).to(self.device), ws))
            self.launches_per_run = 2 * len(self._ta)
            return
        # one grouped launch per sub-batch of at most 8 rows (the row loops' limit)
        with torch.cuda.device(self.device):
            for b0 in range(0, batch, MAX_GEMV_BATCH):
                nb = min(MAX_GEMV_BATCH, batch - b0)
                sub = (_lib.jq_problem * n)()
                ctypes.memmove(sub, arr, ctypes.sizeof(arr))
                for i, (w, nf) in enumerate(zip(weights, self.full_rows)):
                    sub[i].x = arr[i].x + b0 * w.K * esz
                    sub[i].y = arr[i].y + b0 * nf * esz
                nbytes = lib.jq_grouped_plan_bytes(n)
                plan_host = np.zeros((nbytes + 3) // 4, dtype=np.int32)
                _lib.check(lib.jq_grouped_plan(spec0.fmt_id, ctypes.byref(sub), n, nb, plan_host.ctypes.data,
                                               plan_host.nbytes), "jq_grouped_plan")
                raw = np.frombuffer(bytes(sub), dtype=np.uint8).copy()
                self._subs.append((torch.from_numpy(raw).to(self.device), plan_host,
                                   torch.from_numpy(plan_host).to(self.device)))
        self.launches_per_run = len(self._subs)

    @property
    def fused_exchange(self) -> bool:
        return self._symm is not None

    def barrier(self) -> None:
        """Order the ranks after run(): every rank's stores into this rank's
        output arena are complete once this returns on the stream."""
        if self._symm is not None:
            self._symm.barrier()

    def status(self, clear: bool = True) -> int:
        """Sticky device status of the pair-table kernels' workspaces (0 = fine);
        synchronises the stream."""
        lib = _lib.load()
        worst = 0
        with torch.cuda.device(self.device):
            for _, _, ws in self._ta:
                worst = min(worst, lib.jq_ta_status(_ptr(ws), 1 if clear else 0, _stream()))
        return worst

    def run(self) -> None:
        lib = _lib.load()
        if self._ta:
            with torch.cuda.device(self.device):
                for plan_host, plan_dev, ws in self._ta:
                    st = lib.jq_gemm_ta_grouped(plan_host.ctypes.data, _ptr(plan_dev), _ptr(ws), _DT[self.x_dtype],
                                                _DT[self.x_dtype], len(self._peer_delta), self._peer_delta.ctypes.data,
                                                _stream())
                    _lib.check(st, "jq_gemm_ta_grouped")
            return
        if not self._per_problem:
            st = 0
            with torch.cuda.device(self.device):
                for problems_dev, plan_host, plan_dev in self._subs:
                    st = lib.jq_gemv_grouped_peers(_ptr(problems_dev), plan_host.ctypes.data, _ptr(plan_dev),
                                                   _DT[self.x_dtype], _DT[self.x_dtype], len(self._peer_delta),
                                                   self._peer_delta.ctypes.data, _stream())
                    if st:
                        break
            if st != -5:
                _lib.check(st, "jq_gemv_grouped")
                return
            if self._symm is not None:
                _lib.check(st, "jq_gemv_grouped_peers")
            # batch x K too large for one staged activation per CTA: one (split-K) launch per matrix instead
            warnings.warn("GroupedGemv: this batch x K does not fit a grouped launch; running one launch per matrix")
            self._per_problem = True
        for w, x, y, b, nf, ro in zip(self.weights, self.xs, self.ys, self.biases, self.full_rows, self.row_offsets):
            y[:, ro:ro + w.N].copy_(linear(x, w, b))
        self.launches_per_run = None
