"""The reference's three hot-path operators, backed by the sm_100a kernels.

Same names and call signatures as the reference so that hawk/hawk.py can bind them in
place of its own (hawk/hawk.py:12-14):

    fused_linear_scan(x, x_rg_lru, a_rg_lru, a_param) -> h        hawk/scan_fused.py:445
    Conv1D(width, temporal_width, w_init_variance_scale)(x) -> y   hawk/external.py:12-98
    fused_cross_entropy(lm_head_weight, act, labels) -> loss       hawk/fused_cross_entropy.py:77-79

plus the two halves of the cached decode step (hawk/hawk.py:137-151,168-199) and the block's glue in
single passes: gelu(a) * b, RMSNorm with the preceding residual add, the block-diagonal gate pair.

Each op is a torch.library custom op (with a fake/meta kernel and a registered backward), so
torch.compile treats it as an opaque call; the real implementation hands raw device pointers
and the current CUDA stream to the C ABI in libhawk_b200.so.  There is no CPU path: tensors
must live on a CUDA device and the library must have been built.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib

_DT = {torch.float32: _lib.HAWK_F32, torch.bfloat16: _lib.HAWK_BF16}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"hawk_b200: unsupported dtype {t.dtype} (float32 and bfloat16 only)") from None


def _stream(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise RuntimeError("hawk_b200: tensors must be on a CUDA device (there is no CPU path)")
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class KernelLog:
    """Counts the kernels this library launches and, on request, brackets every C-ABI call with CUDA
    events on the launching stream (how the benchmark measures kernel time inside a training step)."""

    def __init__(self):
        self.enabled = False
        self.timed = False
        self.only = None
        self.counts = {}
        self.events = {}

    def reset(self, enabled: bool = True, timed: bool = False, only=None) -> None:
        """`only`: names of the entry points to bracket with events (None = all); counting covers all."""
        self.enabled, self.timed = enabled, timed
        self.only = None if only is None else frozenset(only)
        self.counts, self.events = {}, {}

    def total_launches(self) -> int:
        return sum(self.counts.values())

    def mean_ms(self, name: str) -> Optional[float]:
        """Mean device time of one call of `name` (call after torch.cuda.synchronize())."""
        ev = self.events.get(name)
        if not ev:
            return None
        return sum(a.elapsed_time(b) for a, b in ev) / len(ev)


LOG = KernelLog()


class _on:
    """Makes the tensor's device current for the duration of a C-ABI call (no-op when it already is)
    and reports the call to LOG: `name` is the entry point, `kernels` how many kernels it launches."""

    def __init__(self, t, name: str = "", kernels: int = 0):
        if not t.is_cuda:
            raise RuntimeError("hawk_b200: tensors must be on a CUDA device (there is no CPU path)")
        self.idx = t.device.index
        self.prev = None
        self.name, self.kernels = name, kernels
        self.stream = None
        self.start = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if self.idx is not None and self.idx != cur:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        if LOG.enabled and self.name:
            LOG.counts[self.name] = LOG.counts.get(self.name, 0) + self.kernels
            if LOG.timed and (LOG.only is None or self.name in LOG.only):
                self.stream = torch.cuda.current_stream()
                self.start = torch.cuda.Event(enable_timing=True)
                self.start.record(self.stream)

    def __exit__(self, *a):
        if self.start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record(self.stream)
            LOG.events.setdefault(self.name, []).append((self.start, end))
        if self.prev is not None:
            torch.cuda.set_device(self.prev)


# ---------------------------------------------------------------------------------------------
# RG-LRU scan
# ---------------------------------------------------------------------------------------------
# bytes each entry point must move per [B,T,D] element with bf16 storage (its HBM roofline), and the
# pair of entry points the model's training step launches for the scan
SCAN_BYTES_PER_ELEMENT = {"scan_fwd": 8, "scan_bwd": 16, "scan_gelu_fwd": 12, "scan_gelu_bwd": 20}
SCAN_ENTRY_POINTS = ("scan_gelu_fwd", "scan_gelu_bwd")

def _split_workspace(lib, x, B, nsub, D):
    return torch.empty(lib.hawk_scan_split_workspace_bytes(B, nsub, D), dtype=torch.uint8, device=x.device)


def _split_view_ok(v, T):
    """y / dy of a time-split scan: consecutive sequences exactly T rows apart (or a single sequence)."""
    return v.shape[0] == 1 or v.stride(0) == T * v.stride(1)


@torch.library.custom_op("hawk_b200::scan_fwd", mutates_args=())
def scan_fwd(x: torch.Tensor, gx: torch.Tensor, ga: torch.Tensor, lam: torch.Tensor,
             h0: Optional[torch.Tensor] = None, gate_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = _lib.load()
    B, T, D = x.shape
    x, gx, ga, lam = x.contiguous(), gx.contiguous(), ga.contiguous(), lam.contiguous()
    if h0 is not None:
        h0 = h0.contiguous()
    if gate_bias is not None:
        assert gate_bias.shape == (2, D) and gate_bias.dtype == torch.float32, "gate_bias: [2, D] fp32"
        gate_bias = gate_bias.contiguous()
    h = torch.empty_like(x)
    nsub = lib.hawk_scan_split_chunks(B, T, D, 0)
    if nsub > 1:  # few (sequence, channel group) pairs: cut the sequences so that every SM gets work
        ws = _split_workspace(lib, x, B, nsub, D)
        with _on(x, "scan_fwd_split", 3):
            _lib.check(lib.hawk_scan_fwd_split(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(), _ptr(h0),
                                               _ptr(gate_bias), None, 0, 0, h.data_ptr(), None, nsub, ws.data_ptr(),
                                               ws.numel(), B, T, D, _dt(x), _stream(x)), "hawk_scan_fwd_split")
        return h
    with _on(x, "scan_fwd", 1):
        _lib.check(lib.hawk_scan_fwd(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(), _ptr(h0),
                                     _ptr(gate_bias), h.data_ptr(), B, T, D, _dt(x), _stream(x)), "hawk_scan_fwd")
    return h


@scan_fwd.register_fake
def _(x, gx, ga, lam, h0=None, gate_bias=None):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.custom_op("hawk_b200::scan_bwd", mutates_args=())
def scan_bwd(x: torch.Tensor, gx: torch.Tensor, ga: torch.Tensor, lam: torch.Tensor, h0: Optional[torch.Tensor],
             gate_bias: Optional[torch.Tensor], h: torch.Tensor, go: torch.Tensor
             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(dx, dgx, dga, dlam, dh0, dgate_bias); dgate_bias is [2, D] (empty [0, D] without gate_bias)."""
    lib = _lib.load()
    B, T, D = x.shape
    x, gx, ga, lam, h, go = (t.contiguous() for t in (x, gx, ga, lam, h, go))
    if go.dtype != x.dtype:
        go = go.to(x.dtype)
    dx, dgx, dga = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
    dlam = torch.empty(D, dtype=torch.float32, device=x.device)
    dh0 = torch.empty(B, D, dtype=torch.float32, device=x.device)
    dgb = torch.empty(2 if gate_bias is not None else 0, D, dtype=torch.float32, device=x.device)
    ws_bytes = (3 if gate_bias is not None else 1) * B * D * 4
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    if h0 is not None:
        h0 = h0.contiguous()
    if gate_bias is not None:
        gate_bias = gate_bias.contiguous()
    nsub = lib.hawk_scan_split_chunks(B, T, D, 2)
    if nsub > 1:
        ws = _split_workspace(lib, x, B, nsub, D)
        with _on(x, "scan_bwd_split", 5):
            _lib.check(lib.hawk_scan_bwd_split(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(), _ptr(h0),
                                               _ptr(gate_bias), h.data_ptr(), None, 0, 0, go.data_ptr(), dx.data_ptr(),
                                               dgx.data_ptr(), dga.data_ptr(), None, 0, 0, dlam.data_ptr(),
                                               dh0.data_ptr(), dgb.data_ptr() if gate_bias is not None else None,
                                               nsub, ws.data_ptr(), ws.numel(), B, T, D, _dt(x), _stream(x)),
                       "hawk_scan_bwd_split")
        return dx, dgx, dga, dlam, dh0, dgb
    with _on(x, "scan_bwd", 2):
        _lib.check(lib.hawk_scan_bwd(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(), _ptr(h0),
                                     _ptr(gate_bias), h.data_ptr(), go.data_ptr(), dx.data_ptr(), dgx.data_ptr(),
                                     dga.data_ptr(), dlam.data_ptr(), dh0.data_ptr(),
                                     dgb.data_ptr() if gate_bias is not None else None, ws.data_ptr(), ws_bytes,
                                     B, T, D, _dt(x), _stream(x)), "hawk_scan_bwd")
    return dx, dgx, dga, dlam, dh0, dgb


@scan_bwd.register_fake
def _(x, gx, ga, lam, h0, gate_bias, h, go):
    B, T, D = x.shape
    e = lambda: torch.empty_like(x, memory_format=torch.contiguous_format)
    return (e(), e(), e(), x.new_empty(D, dtype=torch.float32), x.new_empty(B, D, dtype=torch.float32),
            x.new_empty(2 if gate_bias is not None else 0, D, dtype=torch.float32))


def _scan_setup(ctx, inputs, output):
    x, gx, ga, lam, h0, gate_bias = inputs
    ctx.save_for_backward(x, gx, ga, lam, h0, gate_bias, output)
    ctx.has_h0 = h0 is not None
    ctx.has_bias = gate_bias is not None


def _scan_backward(ctx, go):
    x, gx, ga, lam, h0, gate_bias, h = ctx.saved_tensors
    dx, dgx, dga, dlam, dh0, dgb = scan_bwd(x, gx, ga, lam, h0, gate_bias, h, go)
    return dx, dgx, dga, dlam, (dh0 if ctx.has_h0 else None), (dgb if ctx.has_bias else None)


scan_fwd.register_autograd(_scan_backward, setup_context=_scan_setup)


def fused_linear_scan(x, x_rg_lru, a_rg_lru, a_param, *, h0=None, gate_bias=None):
    """h = RG-LRU scan of (x, input-gate pre-activation, recurrence-gate pre-activation, Lambda).

    Drop-in for hawk/scan_fused.py:445.  As in the reference (custom_fwd(cast_inputs=bfloat16),
    scan_fused.py:428) the three activation tensors are taken in bf16 under CUDA autocast and in
    their own dtype otherwise, and h has that dtype.  Lambda and its gradient stay fp32 here (the
    reference rounds Lambda to bf16 under autocast).  Two extensions, both off by default: `h0`
    ([B,D]) is the initial state (the reference's is zero); `gate_bias` ([2,D] fp32: input-gate row,
    recurrence-gate row) is added to the gate pre-activations inside the kernel, so that the caller
    can pass bias-free gate projections and gets the bias gradients from the scan's backward.
    """
    if torch.is_autocast_enabled("cuda"):
        dt = torch.bfloat16
    else:
        dt = x.dtype
    x, x_rg_lru, a_rg_lru = (t if t.dtype == dt else t.to(dt) for t in (x, x_rg_lru, a_rg_lru))
    lam = a_param if a_param.dtype == torch.float32 else a_param.float()
    if h0 is not None and h0.dtype != torch.float32:
        h0 = h0.float()
    if gate_bias is not None and gate_bias.dtype != torch.float32:
        gate_bias = gate_bias.float()
    return scan_fwd(x, x_rg_lru, a_rg_lru, lam, h0, gate_bias)


def sequential_scan_forward(x, x_rg_lru, a_rg_lru, a_param):
    """The reference's host function of the forward (hawk/scan_fused.py:319-360): h for tensors of one dtype, no
    autograd, no autocast handling.  Non-contiguous inputs are copied where the reference asserts."""
    lam = a_param if a_param.dtype == torch.float32 else a_param.float()
    return scan_fwd(x, x_rg_lru, a_rg_lru, lam, None, None)


def sequential_scan_backward(x_saved, x_rg_lru_saved, a_rg_lru_saved, a_param_saved, h_saved, grad_out):
    """The reference's host function of the backward (hawk/scan_fused.py:363-424), same argument order:
    (x_grad, x_rg_lru_grad, a_rg_lru_grad, a_param_grad), the last in a_param's dtype as there (:378,424)."""
    lam = a_param_saved if a_param_saved.dtype == torch.float32 else a_param_saved.float()
    dx, dgx, dga, dlam, _, _ = scan_bwd(x_saved, x_rg_lru_saved, a_rg_lru_saved, lam, None, None, h_saved, grad_out)
    return dx, dgx, dga, dlam.to(a_param_saved.dtype)


def _conv_view(x: torch.Tensor) -> torch.Tensor:
    """x as the kernels can read it in place: [B,T,D], unit channel stride, 16-byte aligned rows."""
    ok = (x.stride(2) == 1 and x.stride(1) % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
          and x.stride(1) >= x.shape[2])
    return x if ok else x.contiguous()


# ---- the scan with the block's epilogue out = gelu(y) * h fused in (hawk/hawk.py:134-135,201) ----
@torch.library.custom_op("hawk_b200::scan_gelu_fwd", mutates_args=())
def scan_gelu_fwd(x: torch.Tensor, gx: torch.Tensor, ga: torch.Tensor, lam: torch.Tensor,
                  gate_bias: Optional[torch.Tensor], y: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(h, gelu(y) * h); y [B,T,D] may be a row-strided view (the y half of the input projection)."""
    lib = _lib.load()
    B, T, D = x.shape
    x, gx, ga, lam = x.contiguous(), gx.contiguous(), ga.contiguous(), lam.contiguous()
    assert y.shape == x.shape and y.dtype == x.dtype
    yv = _conv_view(y)
    if gate_bias is not None:
        assert gate_bias.shape == (2, D) and gate_bias.dtype == torch.float32, "gate_bias: [2, D] fp32"
        gate_bias = gate_bias.contiguous()
    h, out = torch.empty_like(x), torch.empty_like(x)
    nsub = lib.hawk_scan_split_chunks(B, T, D, 1) if _split_view_ok(yv, T) else 1
    if nsub > 1:
        ws = _split_workspace(lib, x, B, nsub, D)
        with _on(x, "scan_gelu_fwd_split", 3):
            _lib.check(lib.hawk_scan_fwd_split(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(), None,
                                               _ptr(gate_bias), yv.data_ptr(), T * yv.stride(1), yv.stride(1),
                                               h.data_ptr(), out.data_ptr(), nsub, ws.data_ptr(), ws.numel(), B, T, D,
                                               _dt(x), _stream(x)), "hawk_scan_fwd_split")
        return h, out
    with _on(x, "scan_gelu_fwd", 1):
        _lib.check(lib.hawk_scan_gelu_fwd(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(), _ptr(gate_bias),
                                          yv.data_ptr(), yv.stride(0), yv.stride(1), h.data_ptr(), out.data_ptr(),
                                          B, T, D, _dt(x), _stream(x)), "hawk_scan_gelu_fwd")
    return h, out


@scan_gelu_fwd.register_fake
def _(x, gx, ga, lam, gate_bias, y):
    e = lambda: torch.empty_like(x, memory_format=torch.contiguous_format)
    return e(), e()


@torch.library.custom_op("hawk_b200::scan_gelu_bwd_into", mutates_args=("dy_out",))
def scan_gelu_bwd_into(x: torch.Tensor, gx: torch.Tensor, ga: torch.Tensor, lam: torch.Tensor,
                       gate_bias: Optional[torch.Tensor], h: torch.Tensor, y: torch.Tensor, dout: torch.Tensor,
                       dy_out: torch.Tensor
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Backward of scan_gelu_fwd from d out: returns (dx, dgx, dga, dlam, dgate_bias) and writes d y into
    `dy_out`, a [B,T,D] view that may be row-strided (e.g. the y half of the projection's gradient)."""
    lib = _lib.load()
    B, T, D = x.shape
    x, gx, ga, lam, h, dout = (t.contiguous() for t in (x, gx, ga, lam, h, dout))
    if dout.dtype != x.dtype:
        dout = dout.to(x.dtype)
    yv = _conv_view(y)
    assert dy_out.shape == x.shape and dy_out.dtype == x.dtype and _conv_view(dy_out) is dy_out
    dx, dgx, dga = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
    dlam = torch.empty(D, dtype=torch.float32, device=x.device)
    dgb = torch.empty(2 if gate_bias is not None else 0, D, dtype=torch.float32, device=x.device)
    ws_bytes = (3 if gate_bias is not None else 1) * B * D * 4
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    if gate_bias is not None:
        gate_bias = gate_bias.contiguous()
    nsub = lib.hawk_scan_split_chunks(B, T, D, 2) if (_split_view_ok(yv, T) and _split_view_ok(dy_out, T)) else 1
    if nsub > 1:
        ws = _split_workspace(lib, x, B, nsub, D)
        with _on(x, "scan_gelu_bwd_split", 5):
            _lib.check(lib.hawk_scan_bwd_split(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(), None,
                                               _ptr(gate_bias), h.data_ptr(), yv.data_ptr(), T * yv.stride(1),
                                               yv.stride(1), dout.data_ptr(), dx.data_ptr(), dgx.data_ptr(),
                                               dga.data_ptr(), dy_out.data_ptr(), T * dy_out.stride(1),
                                               dy_out.stride(1), dlam.data_ptr(), None,
                                               dgb.data_ptr() if gate_bias is not None else None, nsub, ws.data_ptr(),
                                               ws.numel(), B, T, D, _dt(x), _stream(x)), "hawk_scan_bwd_split")
        return dx, dgx, dga, dlam, dgb
    with _on(x, "scan_gelu_bwd", 2):
        _lib.check(lib.hawk_scan_gelu_bwd(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(), _ptr(gate_bias),
                                          h.data_ptr(), yv.data_ptr(), yv.stride(0), yv.stride(1), dout.data_ptr(),
                                          dx.data_ptr(), dgx.data_ptr(), dga.data_ptr(), dy_out.data_ptr(),
                                          dy_out.stride(0), dy_out.stride(1), dlam.data_ptr(),
                                          dgb.data_ptr() if gate_bias is not None else None, ws.data_ptr(), ws_bytes,
                                          B, T, D, _dt(x), _stream(x)), "hawk_scan_gelu_bwd")
    return dx, dgx, dga, dlam, dgb


@scan_gelu_bwd_into.register_fake
def _(x, gx, ga, lam, gate_bias, h, y, dout, dy_out):
    D = x.shape[-1]
    e = lambda: torch.empty_like(x, memory_format=torch.contiguous_format)
    return (e(), e(), e(), x.new_empty(D, dtype=torch.float32),
            x.new_empty(2 if gate_bias is not None else 0, D, dtype=torch.float32))


class _ScanGelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gx, ga, lam, gate_bias, y):
        h, out = scan_gelu_fwd(x, gx, ga, lam, gate_bias, y)
        ctx.save_for_backward(x, gx, ga, lam, gate_bias, y, h)
        ctx.mark_non_differentiable(h)
        ctx.set_materialize_grads(False)
        return out, h

    @staticmethod
    def backward(ctx, dout, _dh):
        if dout is None:
            return (None,) * 6
        x, gx, ga, lam, gate_bias, y, h = ctx.saved_tensors
        dy = torch.empty_like(x)
        dx, dgx, dga, dlam, dgb = scan_gelu_bwd_into(x, gx, ga, lam, gate_bias, h, y, dout, dy)
        return dx, dgx, dga, dlam, (dgb if gate_bias is not None else None), dy


def fused_scan_gelu(x, x_rg_lru, a_rg_lru, a_param, y, *, gate_bias=None):
    """(gelu(y) * h, h) with h = fused_linear_scan(x, x_rg_lru, a_rg_lru, a_param): the RG-LRU scan and the
    recurrent block's epilogue (hawk/hawk.py:134-135,186,201) in one kernel each way.  Dtype rules as
    fused_linear_scan; h is returned for the decode cache and carries no gradient (use out)."""
    dt = torch.bfloat16 if torch.is_autocast_enabled("cuda") else x.dtype
    x, x_rg_lru, a_rg_lru, y = (t if t.dtype == dt else t.to(dt) for t in (x, x_rg_lru, a_rg_lru, y))
    lam = a_param if a_param.dtype == torch.float32 else a_param.float()
    if gate_bias is not None and gate_bias.dtype != torch.float32:
        gate_bias = gate_bias.float()
    return _ScanGelu.apply(x, x_rg_lru, a_rg_lru, lam, gate_bias, y)


# ---------------------------------------------------------------------------------------------
# temporal conv1d
# ---------------------------------------------------------------------------------------------


@torch.library.custom_op("hawk_b200::conv1d_fwd", mutates_args=())
def conv1d_fwd(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    lib = _lib.load()
    B, T, D = x.shape
    xv = _conv_view(x)
    w, b = w.contiguous(), b.contiguous()
    y = torch.empty(B, T, D, dtype=out_dtype, device=x.device)
    with _on(x, "conv1d_fwd", 1):
        _lib.check(lib.hawk_conv1d_fwd(xv.data_ptr(), xv.stride(0), xv.stride(1), w.data_ptr(), b.data_ptr(),
                                       y.data_ptr(), B, T, D, w.shape[0], _dt(xv), _DT[out_dtype], _stream(x)),
                   "hawk_conv1d_fwd")
    return y


@conv1d_fwd.register_fake
def _(x, w, b, out_dtype):
    return x.new_empty(x.shape, dtype=out_dtype)


@torch.library.custom_op("hawk_b200::conv1d_bwd", mutates_args=())
def conv1d_bwd(go: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    B, T, D = x.shape
    W = w.shape[0]
    xv = _conv_view(x)
    go, w = go.contiguous(), w.contiguous()
    dx = torch.empty(B, T, D, dtype=x.dtype, device=x.device)
    dw = torch.empty(W, D, dtype=torch.float32, device=x.device)
    db = torch.empty(D, dtype=torch.float32, device=x.device)
    ws_bytes = lib.hawk_conv1d_bwd_workspace_bytes(B, T, D, W)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    with _on(x, "conv1d_bwd", 2):
        _lib.check(lib.hawk_conv1d_bwd(go.data_ptr(), xv.data_ptr(), xv.stride(0), xv.stride(1), w.data_ptr(),
                                       dx.data_ptr(), dx.stride(0), dx.stride(1), dw.data_ptr(), db.data_ptr(),
                                       ws.data_ptr(), ws_bytes, B, T, D, W, _dt(go), _dt(xv), _stream(x)),
                   "hawk_conv1d_bwd")
    return dx, dw, db


@conv1d_bwd.register_fake
def _(go, x, w):
    return (x.new_empty(x.shape), w.new_empty(w.shape, dtype=torch.float32),
            w.new_empty(w.shape[1], dtype=torch.float32))


def _conv_setup(ctx, inputs, output):
    x, w, b, _ = inputs
    ctx.save_for_backward(x, w)
    ctx.w_dtype, ctx.b_dtype = w.dtype, b.dtype


def _conv_backward(ctx, go):
    x, w = ctx.saved_tensors
    dx, dw, db = conv1d_bwd(go, x, w)
    return dx, dw, db, None


conv1d_fwd.register_autograd(_conv_backward, setup_context=_conv_setup)


@torch.library.custom_op("hawk_b200::conv1d_bwd_into", mutates_args=("dx_out",))
def conv1d_bwd_into(go: torch.Tensor, x: torch.Tensor, w: torch.Tensor,
                    dx_out: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """conv1d_bwd with the input gradient written into `dx_out`, a [B,T,D] view that may be row-strided
    (e.g. one half of the gradient of the projection x was chunked from).  Returns (dw, db)."""
    lib = _lib.load()
    B, T, D = x.shape
    W = w.shape[0]
    xv = _conv_view(x)
    assert dx_out.shape == x.shape and dx_out.dtype == x.dtype and _conv_view(dx_out) is dx_out
    go, w = go.contiguous(), w.contiguous()
    dw = torch.empty(W, D, dtype=torch.float32, device=x.device)
    db = torch.empty(D, dtype=torch.float32, device=x.device)
    ws_bytes = lib.hawk_conv1d_bwd_workspace_bytes(B, T, D, W)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    with _on(x, "conv1d_bwd", 2):
        _lib.check(lib.hawk_conv1d_bwd(go.data_ptr(), xv.data_ptr(), xv.stride(0), xv.stride(1), w.data_ptr(),
                                       dx_out.data_ptr(), dx_out.stride(0), dx_out.stride(1), dw.data_ptr(),
                                       db.data_ptr(), ws.data_ptr(), ws_bytes, B, T, D, W, _dt(go), _dt(xv),
                                       _stream(x)), "hawk_conv1d_bwd")
    return dw, db


@conv1d_bwd_into.register_fake
def _(go, x, w, dx_out):
    return w.new_empty(w.shape, dtype=torch.float32), w.new_empty(w.shape[1], dtype=torch.float32)


def temporal_conv1d(x, w, b, *, out_dtype=None):
    """y[b,t,d] = bias[d] + sum_k w[W-1-k,d] x[b,t-k,d] (zero history).  x may be a strided view.

    out_dtype=None gives the reference's result type (promotion of x and w dtypes: fp32 for a
    bf16 x under autocast, hawk/external.py:88-93); pass x.dtype to have the kernel round on
    store instead of running a separate cast.
    """
    if out_dtype is None:
        out_dtype = torch.promote_types(x.dtype, w.dtype)
    w32 = w if w.dtype == torch.float32 else w.float()
    b32 = b if b.dtype == torch.float32 else b.float()
    return conv1d_fwd(x, w32, b32, out_dtype)


class Conv1D(nn.Module):
    """Drop-in for hawk/external.py:12-150: same constructor, parameter names (`w` [temporal_width,
    width], `b` [width], fp32) and initialisation (external.py:40-47)."""

    def __init__(self, width: int, temporal_width: int, w_init_variance_scale: float = 0.01):
        super().__init__()
        self.width = width
        self.temporal_width = temporal_width
        self.w_init_variance_scale = w_init_variance_scale
        self.w = nn.Parameter(torch.empty([temporal_width, width], dtype=torch.float32))
        self.b = nn.Parameter(torch.empty([width], dtype=torch.float32))
        self.out_dtype = None  # None = reference promotion; set to e.g. torch.bfloat16 to fuse the cast
        nn.init.normal_(self.w, mean=0.0, std=math.sqrt(w_init_variance_scale / temporal_width))
        nn.init.zeros_(self.b)

    def forward(self, x):
        return temporal_conv1d(x, self.w, self.b, out_dtype=self.out_dtype)

    def doc_mask_forward(self, x):
        """The reference's name for the same computation (hawk/external.py:49-95; its forward is this method,
        :97-98; no document mask is applied there either: prompt_len = 0, segment positions unused)."""
        return self.forward(x)


# ---------------------------------------------------------------------------------------------
# cached decode step
# ---------------------------------------------------------------------------------------------
@torch.library.custom_op("hawk_b200::decode_conv_step", mutates_args=("conv_state",))
def decode_conv_step(x_new: torch.Tensor, conv_state: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """x_new [B,D] (row-strided ok), conv_state [B,W-1,D] contiguous, rolled in place. Returns y [B,D]."""
    lib = _lib.load()
    B, D = x_new.shape
    if x_new.stride(1) != 1 or x_new.stride(0) % 8 or x_new.data_ptr() % 16:
        x_new = x_new.contiguous()
    assert conv_state.is_contiguous() and conv_state.shape == (B, w.shape[0] - 1, D)
    y = torch.empty(B, D, dtype=x_new.dtype, device=x_new.device)
    with _on(x_new, "decode_conv_step", 1):
        _lib.check(lib.hawk_decode_conv_step(x_new.data_ptr(), x_new.stride(0), conv_state.data_ptr(), w.data_ptr(),
                                             b.data_ptr(), y.data_ptr(), B, D, w.shape[0], _dt(x_new),
                                             _dt(conv_state), _stream(x_new)), "hawk_decode_conv_step")
    return y


@decode_conv_step.register_fake
def _(x_new, conv_state, w, b):
    return x_new.new_empty(x_new.shape)


@torch.library.custom_op("hawk_b200::decode_block_step", mutates_args=("conv_state", "state"))
def decode_block_step(xy: torch.Tensor, conv_state: torch.Tensor, conv_w: torch.Tensor, conv_b: torch.Tensor,
                      wx: torch.Tensor, wa: torch.Tensor, bx: torch.Tensor, ba: torch.Tensor, lam: torch.Tensor,
                      state: torch.Tensor) -> torch.Tensor:
    """One cached token through the whole recurrent branch in one launch: xy [B,2R] = [x_b | y] (row-strided
    ok), conv_state [B,W-1,R] and state [B,R] updated in place, gate weights [nb,bw,bw] (fp32 or bf16),
    biases / conv taps / Lambda fp32.  Returns gelu(y) * h, [B,R] in xy's dtype."""
    lib = _lib.load()
    B, R2 = xy.shape
    R = R2 // 2
    nb, bw, _ = wx.shape
    if xy.stride(1) != 1:
        xy = xy.contiguous()
    assert conv_state.is_contiguous() and state.is_contiguous() and state.shape == (B, R)
    assert conv_state.dtype == state.dtype and wx.dtype == wa.dtype and nb * bw == R
    wx, wa, bx, ba = wx.contiguous(), wa.contiguous(), bx.contiguous(), ba.contiguous()
    out = torch.empty(B, R, dtype=xy.dtype, device=xy.device)
    with _on(xy, "decode_block_step", 1):
        _lib.check(lib.hawk_decode_block_step(xy.data_ptr(), xy.stride(0), conv_state.data_ptr(), conv_w.data_ptr(),
                                              conv_b.data_ptr(), wx.data_ptr(), wa.data_ptr(), bx.data_ptr(),
                                              ba.data_ptr(), lam.data_ptr(), state.data_ptr(), out.data_ptr(), B, R,
                                              bw, conv_w.shape[0], _dt(xy), _dt(state), _dt(wx), _stream(xy)),
                   "hawk_decode_block_step")
    return out


@decode_block_step.register_fake
def _(xy, conv_state, conv_w, conv_b, wx, wa, bx, ba, lam, state):
    return xy.new_empty(xy.shape[0], xy.shape[1] // 2)


@torch.library.custom_op("hawk_b200::decode_rglru_step", mutates_args=("state",))
def decode_rglru_step(x: torch.Tensor, gx: torch.Tensor, ga: torch.Tensor, lam: torch.Tensor,
                      state: torch.Tensor) -> torch.Tensor:
    """One recurrence step on [B,D]; `state` is overwritten with h; returns h in x's dtype."""
    lib = _lib.load()
    B, D = x.shape
    x, gx, ga = x.contiguous(), gx.contiguous(), ga.contiguous()
    assert state.is_contiguous() and state.shape == (B, D)
    h = torch.empty_like(x)
    with _on(x, "decode_rglru_step", 1):
        _lib.check(lib.hawk_decode_rglru_step(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(),
                                              state.data_ptr(), h.data_ptr(), B, D, _dt(x), _dt(state), _stream(x)),
                   "hawk_decode_rglru_step")
    return h


@decode_rglru_step.register_fake
def _(x, gx, ga, lam, state):
    return torch.empty_like(x)


# ---------------------------------------------------------------------------------------------
# fused linear + cross-entropy
# ---------------------------------------------------------------------------------------------
_ce_status = {}  # device index -> int32[1] status word shared by every call on that device


def _status_word(device: torch.device) -> torch.Tensor:
    t = _ce_status.get(device.index)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _ce_status[device.index] = t
    return t


def check_device_status(device=None) -> None:
    """Raises if a kernel on `device` gave up a bounded wait since the last check (synchronises)."""
    for idx, t in list(_ce_status.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        if int(t.item()) != 0:
            t.zero_()
            raise RuntimeError("hawk_b200: a tcgen05 GEMM abandoned a bounded mbarrier wait; results are invalid")


@torch.library.custom_op("hawk_b200::linear_ce", mutates_args=())
def linear_ce(weight: torch.Tensor, act: torch.Tensor, labels: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(loss [], dweight [V,H] fp32, dact [N,H] fp32) of mean CE(act @ weight^T, labels)."""
    lib = _lib.load()
    V, H = weight.shape
    N = act.shape[0]
    weight, act, labels = weight.contiguous(), act.contiguous(), labels.contiguous()
    if labels.dtype != torch.int64:
        labels = labels.long()
    loss = torch.empty((), dtype=torch.float32, device=act.device)
    dweight = torch.empty(V, H, dtype=torch.float32, device=act.device)
    dact = torch.empty(N, H, dtype=torch.float32, device=act.device)
    ws_bytes = lib.hawk_linear_ce_workspace_bytes(N, H, V)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=act.device)
    with _on(act, "linear_ce", 9 if weight.dtype == torch.float32 else 7):
        _lib.check(lib.hawk_linear_ce_fwd_bwd(weight.data_ptr(), act.data_ptr(), labels.data_ptr(), loss.data_ptr(),
                                              dweight.data_ptr(), dact.data_ptr(), ws.data_ptr(), ws_bytes, N, H, V,
                                              _dt(weight), _status_word(act.device).data_ptr(), _stream(act)),
                   "hawk_linear_ce_fwd_bwd")
    return loss, dweight, dact


@linear_ce.register_fake
def _(weight, act, labels):
    return (act.new_empty((), dtype=torch.float32), weight.new_empty(weight.shape, dtype=torch.float32),
            act.new_empty(act.shape, dtype=torch.float32))


def _ce_setup(ctx, inputs, output):
    weight, act, _ = inputs
    _, dweight, dact = output
    ctx.save_for_backward(dweight, dact)
    ctx.dtypes = (weight.dtype, act.dtype)


def _ce_backward(ctx, g_loss, g_dw, g_da):
    dweight, dact = ctx.saved_tensors  # computed in the forward, as in the reference (:63,66-73)
    wd, ad = ctx.dtypes
    return (g_loss * dweight).to(wd), (g_loss * dact).to(ad), None


linear_ce.register_autograd(_ce_backward, setup_context=_ce_setup)


def fused_cross_entropy(lm_head_weight, act, labels):
    """Mean cross-entropy of `act @ lm_head_weight.T` against `labels`; drop-in for
    hawk/fused_cross_entropy.py:77-79.  weight [V,H], act [N,H] (fp32 or bf16), labels [N] int64.
    The arithmetic is the reference's under bf16 autocast whether or not autocast is on: bf16
    tensor-core GEMMs with fp32 accumulation, bf16 logits, fp32 softmax."""
    if act.dtype != lm_head_weight.dtype:
        act = act.to(lm_head_weight.dtype)
    return linear_ce(lm_head_weight, act, labels)[0]


class CrossEntropyLoopedFused:
    """The reference's autograd class by name (hawk/fused_cross_entropy.py:11-73): `.apply(weight, act, labels)`
    is fused_cross_entropy (one pass over all rows here, no chunk loop)."""
    apply = staticmethod(fused_cross_entropy)


class DiagonalRecurrence:
    """The reference's autograd class by name (hawk/scan_fused.py:426-442): `.apply(x, x_rg_lru, a_rg_lru, a_param)`
    is fused_linear_scan (:445)."""
    apply = staticmethod(fused_linear_scan)


# ---------------------------------------------------------------------------------------------
# glue around the GEMMs: gelu(a) * b and RMSNorm, one pass each
# ---------------------------------------------------------------------------------------------
def _as_rows(t: torch.Tensor):
    """(tensor, M, pitch): t viewed as M rows of t.shape[-1] contiguous elements with one row pitch
    (in elements), in place when its strides allow (e.g. a chunk of a projection output)."""
    J = t.shape[-1]
    M = t.numel() // J if J else 0
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0
    if ok and t.dim() >= 2:
        ld = t.stride(-2)
        expect = ld
        for d in range(t.dim() - 2, -1, -1):  # leading dims must collapse onto the row pitch
            if t.shape[d] != 1 and t.stride(d) != expect:
                ok = False
                break
            expect = t.stride(d) * t.shape[d]
        ok = ok and ld % 8 == 0 and ld >= J
    elif ok:
        ld = J
    if not ok:
        t = t.contiguous()
        ld = J
    return t, M, ld


@torch.library.custom_op("hawk_b200::gelu_mul_fwd", mutates_args=())
def gelu_mul_fwd(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    lib = _lib.load()
    av, M, lda = _as_rows(a)
    bv, _, ldb = _as_rows(b)
    out = torch.empty(a.shape, dtype=a.dtype, device=a.device)
    with _on(a, "gelu_mul_fwd", 1):
        _lib.check(lib.hawk_gelu_mul_fwd(av.data_ptr(), lda, bv.data_ptr(), ldb, out.data_ptr(), a.shape[-1], M,
                                         a.shape[-1], _dt(a), _stream(a)), "hawk_gelu_mul_fwd")
    return out


@gelu_mul_fwd.register_fake
def _(a, b):
    return a.new_empty(a.shape)


@torch.library.custom_op("hawk_b200::gelu_mul_bwd", mutates_args=())
def gelu_mul_bwd(dout: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    J = a.shape[-1]
    av, M, lda = _as_rows(a)
    bv, _, ldb = _as_rows(b)
    dv, _, ldd = _as_rows(dout)
    da = torch.empty(a.shape, dtype=a.dtype, device=a.device)
    db = torch.empty(a.shape, dtype=a.dtype, device=a.device)
    with _on(a, "gelu_mul_bwd", 1):
        _lib.check(lib.hawk_gelu_mul_bwd(dv.data_ptr(), ldd, av.data_ptr(), lda, bv.data_ptr(), ldb, da.data_ptr(), J,
                                         db.data_ptr(), J, M, J, _dt(a), _stream(a)), "hawk_gelu_mul_bwd")
    return da, db


@gelu_mul_bwd.register_fake
def _(dout, a, b):
    return a.new_empty(a.shape), a.new_empty(a.shape)


@torch.library.custom_op("hawk_b200::gelu_mul_bwd_into", mutates_args=("da_out",))
def gelu_mul_bwd_into(dout: torch.Tensor, a: torch.Tensor, b: torch.Tensor, da_out: torch.Tensor) -> torch.Tensor:
    """gelu_mul_bwd with d a written into `da_out` (same shape as a; may be a row-strided view such as
    one half of a wider gradient buffer).  Returns d b."""
    lib = _lib.load()
    J = a.shape[-1]
    av, M, lda = _as_rows(a)
    bv, _, ldb = _as_rows(b)
    dv, _, ldd = _as_rows(dout)
    ov, _, ldo = _as_rows(da_out)
    assert ov is da_out and da_out.shape == a.shape and da_out.dtype == a.dtype, "da_out must be usable in place"
    db = torch.empty(a.shape, dtype=a.dtype, device=a.device)
    with _on(a, "gelu_mul_bwd", 1):
        _lib.check(lib.hawk_gelu_mul_bwd(dv.data_ptr(), ldd, av.data_ptr(), lda, bv.data_ptr(), ldb, ov.data_ptr(), ldo,
                                         db.data_ptr(), J, M, J, _dt(a), _stream(a)), "hawk_gelu_mul_bwd")
    return db


@gelu_mul_bwd_into.register_fake
def _(dout, a, b, da_out):
    return a.new_empty(a.shape)


def _gm_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _gm_backward(ctx, dout):
    a, b = ctx.saved_tensors
    return gelu_mul_bwd(dout, a, b)


gelu_mul_fwd.register_autograd(_gm_backward, setup_context=_gm_setup)


def gelu_mul(a, b):
    """gelu(a) * b (exact GELU) in one pass; a and b may be strided halves of a projection output."""
    if b.dtype != a.dtype:
        b = b.to(a.dtype)
    return gelu_mul_fwd(a, b)


@torch.library.custom_op("hawk_b200::geglu_fwd", mutates_args=())
def geglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    """gelu(gu[..., :I]) * gu[..., I:] for a contiguous [.., 2I] projection output."""
    lib = _lib.load()
    gu = gu.contiguous()
    I = gu.shape[-1] // 2
    M = gu.numel() // (2 * I)
    out = torch.empty(*gu.shape[:-1], I, dtype=gu.dtype, device=gu.device)
    es = gu.element_size()
    with _on(gu, "gelu_mul_fwd", 1):
        _lib.check(lib.hawk_gelu_mul_fwd(gu.data_ptr(), 2 * I, gu.data_ptr() + I * es, 2 * I, out.data_ptr(), I, M, I,
                                         _dt(gu), _stream(gu)), "hawk_gelu_mul_fwd")
    return out


@geglu_fwd.register_fake
def _(gu):
    return gu.new_empty(*gu.shape[:-1], gu.shape[-1] // 2)


@torch.library.custom_op("hawk_b200::geglu_bwd", mutates_args=())
def geglu_bwd(dout: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    """Gradient of geglu_fwd w.r.t. gu: both halves written straight into one [.., 2I] buffer."""
    lib = _lib.load()
    gu, dout = gu.contiguous(), dout.contiguous()
    I = gu.shape[-1] // 2
    M = gu.numel() // (2 * I)
    dgu = torch.empty_like(gu)
    es = gu.element_size()
    with _on(gu, "gelu_mul_bwd", 1):
        _lib.check(lib.hawk_gelu_mul_bwd(dout.data_ptr(), I, gu.data_ptr(), 2 * I, gu.data_ptr() + I * es, 2 * I,
                                         dgu.data_ptr(), 2 * I, dgu.data_ptr() + I * es, 2 * I, M, I, _dt(gu),
                                         _stream(gu)), "hawk_gelu_mul_bwd")
    return dgu


@geglu_bwd.register_fake
def _(dout, gu):
    return torch.empty_like(gu)


geglu_fwd.register_autograd(lambda ctx, dout: geglu_bwd(dout, ctx.saved_tensors[0]),
                            setup_context=lambda ctx, inputs, output: ctx.save_for_backward(inputs[0]))


def geglu(gu):
    """gelu(gate) * up for gu = [gate | up] (hawk/hawk.py:82-86)."""
    return geglu_fwd(gu)


@torch.library.custom_op("hawk_b200::rms_norm_fwd", mutates_args=())
def rms_norm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    x, w = x.contiguous(), w.contiguous()
    H = x.shape[-1]
    M = x.numel() // H
    y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    with _on(x, "rms_norm_fwd", 1):
        _lib.check(lib.hawk_rms_norm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), M, H, eps, _dt(x),
                                         _DT[out_dtype], _stream(x)), "hawk_rms_norm_fwd")
    return y, rstd


@rms_norm_fwd.register_fake
def _(x, w, eps, out_dtype):
    return x.new_empty(x.shape, dtype=out_dtype), x.new_empty(x.numel() // x.shape[-1], dtype=torch.float32)


@torch.library.custom_op("hawk_b200::rms_norm_bwd", mutates_args=())
def rms_norm_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    dy, x, w = dy.contiguous(), x.contiguous(), w.contiguous()
    H = x.shape[-1]
    M = x.numel() // H
    dx = torch.empty_like(x)
    dw = torch.empty(H, dtype=torch.float32, device=x.device)
    ws_bytes = lib.hawk_rms_norm_bwd_workspace_bytes(H)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    with _on(x, "rms_norm_bwd", 2):
        _lib.check(lib.hawk_rms_norm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                         dw.data_ptr(), ws.data_ptr(), ws_bytes, M, H, _dt(x), _dt(dy), _stream(x)),
                   "hawk_rms_norm_bwd")
    return dx, dw


@rms_norm_bwd.register_fake
def _(dy, x, w, rstd):
    return torch.empty_like(x), w.new_empty(w.shape, dtype=torch.float32)


def _rn_setup(ctx, inputs, output):
    x, w, _, _ = inputs
    ctx.save_for_backward(x, w, output[1])
    ctx.w_dtype = w.dtype


def _rn_backward(ctx, dy, drstd):
    x, w, rstd = ctx.saved_tensors
    dx, dw = rms_norm_bwd(dy, x, w, rstd)
    return dx, dw.to(ctx.w_dtype), None, None


rms_norm_fwd.register_autograd(_rn_backward, setup_context=_rn_setup)


def rms_norm(x, weight, eps: float = 1e-6, out_dtype=None):
    """x * rsqrt(mean(x^2) + eps) * weight with fp32 statistics (hawk/hawk.py:47-58).  out_dtype=None
    keeps x's dtype; under autocast the model asks for bf16, which is what the following Linear would
    round its input to anyway."""
    w32 = weight if weight.dtype == torch.float32 else weight.float()
    return rms_norm_fwd(x, w32, eps, out_dtype or x.dtype)[0]


# ---------------------------------------------------------------------------------------------
# both block-diagonal gate projections of the recurrent block, without layout copies
# ---------------------------------------------------------------------------------------------
class _BlockDiagGates(torch.autograd.Function):
    """gx = blockdiag(x; wx) + bx, ga = blockdiag(x; wa) + ba (hawk/external.py:224-233, called twice
    at hawk/hawk.py:181-182).  The [M, nb*bw] activations are used as nb strided batches in place
    (batch stride bw, row pitch nb*bw): cuBLAS strided-batch GEMMs read and write the final layout,
    so no transposed copies are made in either direction."""

    @staticmethod
    def forward(ctx, x, wx, bx, wa, ba):
        nb, bw, _ = wx.shape
        R = nb * bw
        shape = x.shape
        x2 = x.reshape(-1, R)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        dt = x2.dtype
        with torch.autocast("cuda", enabled=False):
            xb = x2.view(M, nb, bw).transpose(0, 1)  # [nb, M, bw] view
            out = torch.empty(2, M, R, dtype=dt, device=x.device)
            wxc, wac = wx.to(dt), wa.to(dt)
            ox, oa = (out[j].view(M, nb, bw).transpose(0, 1) for j in (0, 1))
            if bx is None:  # the caller adds the biases downstream (inside the scan kernel)
                torch.bmm(xb, wxc, out=ox)
                torch.bmm(xb, wac, out=oa)
            else:
                torch.baddbmm(bx.to(dt).unsqueeze(1), xb, wxc, out=ox)
                torch.baddbmm(ba.to(dt).unsqueeze(1), xb, wac, out=oa)
        ctx.save_for_backward(x2, wxc, wac)
        ctx.meta = (shape, nb, bw, wx.dtype, None if bx is None else bx.dtype)
        return out[0].view(shape), out[1].view(shape)

    @staticmethod
    def backward(ctx, dgx, dga):
        x2, wxc, wac = ctx.saved_tensors
        shape, nb, bw, wdt, bdt = ctx.meta
        M, R = x2.shape
        dt = x2.dtype
        with torch.autocast("cuda", enabled=False):
            dgx2 = dgx.reshape(M, R).to(dt).contiguous()
            dga2 = dga.reshape(M, R).to(dt).contiguous()
            gxb = dgx2.view(M, nb, bw).transpose(0, 1)
            gab = dga2.view(M, nb, bw).transpose(0, 1)
            xbT = x2.view(M, nb, bw).permute(1, 2, 0)  # [nb, bw, M] view
            dwx = torch.bmm(xbT, gxb)
            dwa = torch.bmm(xbT, gab)
            dbx = dba = None
            if bdt is not None:
                dbx = dgx2.view(M, nb, bw).sum(dim=0, dtype=torch.float32).to(bdt)
                dba = dga2.view(M, nb, bw).sum(dim=0, dtype=torch.float32).to(bdt)
            dx = torch.empty(M, R, dtype=dt, device=x2.device)
            dxb = dx.view(M, nb, bw).transpose(0, 1)
            torch.bmm(gxb, wxc.transpose(1, 2), out=dxb)
            torch.baddbmm(dxb, gab, wac.transpose(1, 2), out=dxb)
        return dx.view(shape), dwx.to(wdt), dbx, dwa.to(wdt), dba


def block_diag_gates(x, wx, bx, wa, ba):
    """(input-gate, recurrence-gate) pre-activations of the RG-LRU from the conv output x [..., R].
    With bx = ba = None the projections are returned without their biases, for a caller that hands
    the biases to `fused_linear_scan(..., gate_bias=)`."""
    assert (bx is None) == (ba is None)
    return _BlockDiagGates.apply(x, wx, bx, wa, ba)


# ---- the same two projections as one tcgen05 kernel per direction --------------------------------
# bf16 bytes per [M, R] element: forward reads xc, writes gx, ga; backward reads xc, dgx, dga (the latter two
# twice: input- and weight-gradient kernels) and reads + writes dxc
GATE_BYTES_PER_ELEMENT = {"gates_fwd": 6, "gates_bwd": 14}


def gates_kernel_ok(x: torch.Tensor, nb: int, bw: int) -> bool:
    """Whether the fused gate kernels take this case: bf16 activations, block width dividing 128, width a
    multiple of 128 (anything else runs the strided-batch cuBLAS form above)."""
    R = nb * bw
    return x.is_cuda and x.dtype == torch.bfloat16 and R % 128 == 0 and 8 <= bw <= 128 and 128 % bw == 0


@torch.library.custom_op("hawk_b200::gates_pack", mutates_args=())
def gates_pack(wx: torch.Tensor, wa: torch.Tensor) -> torch.Tensor:
    """Both gate weights [nb, bw, bw] (fp32 or bf16) in the operand layouts of gates_fwd / gates_bwd (bf16)."""
    lib = _lib.load()
    nb, bw, _ = wx.shape
    wx, wa = wx.contiguous(), wa.contiguous()
    assert wa.shape == wx.shape and wa.dtype == wx.dtype
    packed = torch.empty(lib.hawk_gates_packed_bytes(nb * bw, bw) // 2, dtype=torch.bfloat16, device=wx.device)
    with _on(wx, "gates_pack", 1):
        _lib.check(lib.hawk_gates_pack_weights(wx.data_ptr(), wa.data_ptr(), _dt(wx), packed.data_ptr(), nb * bw, bw,
                                               _stream(wx)), "hawk_gates_pack_weights")
    return packed


@gates_pack.register_fake
def _(wx, wa):
    nb, bw, _ = wx.shape
    return wx.new_empty((nb * bw // 128) * (256 * 128 + 128 * 384), dtype=torch.bfloat16)


@torch.library.custom_op("hawk_b200::gates_fwd", mutates_args=())
def gates_fwd(xc: torch.Tensor, packed: torch.Tensor, bw: int) -> torch.Tensor:
    """[2, M, R]: (input-gate, recurrence-gate) projections of xc [M, R] bf16, without biases."""
    lib = _lib.load()
    xc = xc.contiguous()
    M, R = xc.shape
    out = torch.empty(2, M, R, dtype=xc.dtype, device=xc.device)
    with _on(xc, "gates_fwd", 1):
        _lib.check(lib.hawk_gates_fwd(xc.data_ptr(), packed.data_ptr(), out[0].data_ptr(), out[1].data_ptr(), M, R, bw,
                                      _status_word(xc.device).data_ptr(), _stream(xc)), "hawk_gates_fwd")
    return out


@gates_fwd.register_fake
def _(xc, packed, bw):
    return xc.new_empty(2, xc.shape[0], xc.shape[1])


@torch.library.custom_op("hawk_b200::gates_bwd_into", mutates_args=("dxc",))
def gates_bwd_into(xc: torch.Tensor, dgx: torch.Tensor, dga: torch.Tensor, packed: torch.Tensor, dxc: torch.Tensor,
                   bw: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """dxc += dgx Wx^T + dga Wa^T in place (dxc [M, R] bf16 contiguous); returns (dwx, dwa) [nb, bw, bw] fp32."""
    lib = _lib.load()
    xc, dgx, dga = xc.contiguous(), dgx.contiguous(), dga.contiguous()
    M, R = xc.shape
    assert dxc.is_contiguous() and dxc.shape == xc.shape and dxc.dtype == xc.dtype
    nb = R // bw
    dwx = torch.empty(nb, bw, bw, dtype=torch.float32, device=xc.device)
    dwa = torch.empty(nb, bw, bw, dtype=torch.float32, device=xc.device)
    ws_bytes = lib.hawk_gates_bwd_workspace_bytes(M, R, bw)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=xc.device)
    with _on(xc, "gates_bwd", 3):
        _lib.check(lib.hawk_gates_bwd(xc.data_ptr(), dgx.data_ptr(), dga.data_ptr(), packed.data_ptr(), dxc.data_ptr(),
                                      dwx.data_ptr(), dwa.data_ptr(), ws.data_ptr(), ws_bytes, M, R, bw,
                                      _status_word(xc.device).data_ptr(), _stream(xc)), "hawk_gates_bwd")
    return dwx, dwa


@gates_bwd_into.register_fake
def _(xc, dgx, dga, packed, dxc, bw):
    nb = xc.shape[1] // bw
    return (xc.new_empty(nb, bw, bw, dtype=torch.float32), xc.new_empty(nb, bw, bw, dtype=torch.float32))


# The strided-batch cuBLAS form of the same two projections for the cases the kernels do not take (fp32
# activations, widths that are not multiples of 128), as opaque operators so that torch.compile traces
# through the recurrent core without looking inside.
@torch.library.custom_op("hawk_b200::gates_bmm_fwd", mutates_args=())
def gates_bmm_fwd(xc: torch.Tensor, wx: torch.Tensor, wa: torch.Tensor) -> torch.Tensor:
    """[2, M, R] from xc [M, R] and weights [nb, bw, bw] already in xc's dtype; reads and writes the final
    layout in place (batch stride bw, row pitch R): no transposed copies."""
    M, R = xc.shape
    nb, bw, _ = wx.shape
    out = torch.empty(2, M, R, dtype=xc.dtype, device=xc.device)
    xb = xc.view(M, nb, bw).transpose(0, 1)  # [nb, M, bw] view
    torch.bmm(xb, wx, out=out[0].view(M, nb, bw).transpose(0, 1))
    torch.bmm(xb, wa, out=out[1].view(M, nb, bw).transpose(0, 1))
    return out


@gates_bmm_fwd.register_fake
def _(xc, wx, wa):
    return xc.new_empty(2, xc.shape[0], xc.shape[1])


@torch.library.custom_op("hawk_b200::gates_bmm_bwd_into", mutates_args=("dxc",))
def gates_bmm_bwd_into(xc: torch.Tensor, dgx: torch.Tensor, dga: torch.Tensor, wx: torch.Tensor, wa: torch.Tensor,
                       dxc: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """dxc += dgx Wx^T + dga Wa^T in place; returns (dwx, dwa) in the weights' dtype."""
    M, R = xc.shape
    nb, bw, _ = wx.shape
    gxb = dgx.view(M, nb, bw).transpose(0, 1)
    gab = dga.view(M, nb, bw).transpose(0, 1)
    xT = xc.view(M, nb, bw).permute(1, 2, 0)  # [nb, bw, M] view
    dwx = torch.bmm(xT, gxb)
    dwa = torch.bmm(xT, gab)
    dxb = dxc.view(M, nb, bw).transpose(0, 1)
    torch.baddbmm(dxb, gxb, wx.transpose(1, 2), out=dxb)
    torch.baddbmm(dxb, gab, wa.transpose(1, 2), out=dxb)
    return dwx, dwa


@gates_bmm_bwd_into.register_fake
def _(xc, dgx, dga, wx, wa, dxc):
    return wx.new_empty(wx.shape), wx.new_empty(wx.shape)


class _FusedGates(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wx, wa):
        nb, bw, _ = wx.shape
        x2 = x.reshape(-1, nb * bw)
        packed = gates_pack(wx.detach(), wa.detach())
        out = gates_fwd(x2, packed, bw)
        ctx.save_for_backward(x2, packed)
        ctx.meta = (x.shape, bw, wx.dtype)
        return out[0].view(x.shape), out[1].view(x.shape)

    @staticmethod
    def backward(ctx, dgx, dga):
        x2, packed = ctx.saved_tensors
        shape, bw, wdt = ctx.meta
        dx = torch.zeros_like(x2)
        dwx, dwa = gates_bwd_into(x2, dgx.reshape(x2.shape).to(x2.dtype), dga.reshape(x2.shape).to(x2.dtype), packed,
                                  dx, bw)
        return dx.view(shape), dwx.to(wdt), dwa.to(wdt)


def fused_block_diag_gates(x, wx, wa):
    """(input-gate, recurrence-gate) projections of x [..., R] WITHOUT biases by the fused kernels (see
    gates_kernel_ok for the cases they take); differentiable in x, wx, wa."""
    nb, bw, _ = wx.shape
    if not gates_kernel_ok(x, nb, bw):
        raise RuntimeError("hawk_b200: fused gate kernels need bf16 activations, block width dividing 128 and "
                           "a width that is a multiple of 128")
    return _FusedGates.apply(x, wx, wa)


# ---------------------------------------------------------------------------------------------
# bf16 projection of an fp32 parameter (what autocast makes of nn.Linear), with fewer passes
# ---------------------------------------------------------------------------------------------
@torch.library.custom_op("hawk_b200::cast_bf16", mutates_args=())
def cast_bf16(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> bf16 copy of a contiguous tensor in one vectorised pass."""
    lib = _lib.load()
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    if x.numel():
        with _on(x, "cast_bf16", 1):
            _lib.check(lib.hawk_cast_f32_bf16(x.data_ptr(), out.data_ptr(), x.numel(), _stream(x)), "hawk_cast_f32_bf16")
    return out


@cast_bf16.register_fake
def _(x):
    return x.new_empty(x.shape, dtype=torch.bfloat16)


class _AutocastLinear(torch.autograd.Function):
    """y = x @ w^T with bf16 operands and fp32 accumulation for an fp32 weight: the arithmetic of
    F.linear under CUDA autocast (hawk/hawk.py:75-86,110-116 run under torch.autocast), minus two
    passes per weight per step: the weight is cast by one vectorised kernel (torch's type-converting
    copy runs at a third of the HBM rate), and the weight gradient leaves its GEMM in fp32 instead of
    being written in bf16 and cast afterwards (so it is also a little more precise than the reference's)."""

    @staticmethod
    def forward(ctx, x, w, wb):
        with torch.autocast("cuda", enabled=False):
            xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
            if wb is None:  # no up-to-date bf16 copy from the optimiser: cast now
                wb = cast_bf16(w.detach())
            y = F.linear(xb, wb)
        ctx.save_for_backward(xb, wb)
        ctx.x_dtype = x.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xb, wb = ctx.saved_tensors
        dx = dw = None
        with torch.autocast("cuda", enabled=False):
            dy2 = dy.reshape(-1, dy.shape[-1])
            if dy2.dtype != torch.bfloat16:
                dy2 = dy2.to(torch.bfloat16)
            if ctx.needs_input_grad[0]:
                dx = torch.mm(dy2, wb).view(xb.shape)
                if dx.dtype != ctx.x_dtype:
                    dx = dx.to(ctx.x_dtype)
            if ctx.needs_input_grad[1]:
                dw = torch.mm(dy2.t(), xb.reshape(-1, xb.shape[-1]), out_dtype=torch.float32)
        return dx, dw, None


def linear(x, w, w_bf16=None):
    """F.linear(x, w) without bias.  Under CUDA autocast with an fp32 weight it runs as `_AutocastLinear`
    (`w_bf16`: an up-to-date bf16 copy of w, e.g. the one `FusedAdamW` writes; cast here when None);
    anywhere else it is F.linear itself."""
    if (x.is_cuda and w.dtype == torch.float32 and torch.is_autocast_enabled("cuda")
            and torch.get_autocast_dtype("cuda") == torch.bfloat16):
        return _AutocastLinear.apply(x, w, w_bf16)
    return F.linear(x, w)


# ---------------------------------------------------------------------------------------------
# the recurrent branch between its two projections as one autograd node
# ---------------------------------------------------------------------------------------------
class _RecurrentCore(torch.autograd.Function):
    """out = gelu(y) * scan(conv(x_b), gates(conv(x_b))) for xy = [x_b | y] (hawk/hawk.py:164-166,
    181-199), and h.  The scan kernels carry the gelu(y) * h epilogue; what one node adds is the
    backward's bookkeeping: d y and d x_b are written straight into the two halves of d xy (no
    concatenation pass for the chunk), and the gate projections accumulate their input gradient onto
    the scan's (no separate add pass)."""

    @staticmethod
    def forward(ctx, xy, conv_w, conv_b, wx, wa, gate_bias, lam):
        R = xy.shape[-1] // 2
        nb, bw, _ = wx.shape
        with torch.autocast("cuda", enabled=False):
            # strides only (traceable by torch.compile); the operators below copy a misaligned view themselves
            if not (xy.stride(-1) == 1 and xy.stride(-2) % 8 == 0 and xy.stride(0) % 8 == 0 and xy.dim() == 3):
                xy = xy.contiguous()
            xb, y = xy[..., :R], xy[..., R:]
            dt = xy.dtype
            xc = conv1d_fwd(xb, conv_w, conv_b, dt)
            M = xc.numel() // R
            fused = gates_kernel_ok(xc, nb, bw)
            if fused:  # both projections in one tcgen05 kernel
                wxc = gates_pack(wx.detach(), wa.detach())
                wac = wxc
                gates = gates_fwd(xc.view(M, R), wxc, bw)
            else:      # strided-batch cuBLAS GEMMs on the final layout
                wxc, wac = wx.to(dt), wa.to(dt)
                gates = gates_bmm_fwd(xc.view(M, R), wxc, wac)
            gx, ga = gates[0].view(xc.shape), gates[1].view(xc.shape)
            h, out = scan_gelu_fwd(xc, gx, ga, lam, gate_bias, y)  # scan and gelu(y) * h in one kernel
        ctx.save_for_backward(xy, conv_w, xc, wxc, wac, gx, ga, lam, gate_bias, h)
        ctx.meta = (nb, bw, conv_w.dtype, conv_b.dtype, wx.dtype, fused)
        ctx.mark_non_differentiable(h)
        ctx.set_materialize_grads(False)  # no zero-filled [B,T,R] gradient for h on every backward
        return out, h

    @staticmethod
    def backward(ctx, dout, _dh):
        if dout is None:
            return (None,) * 7
        xy, conv_w, xc, wxc, wac, gx, ga, lam, gate_bias, h = ctx.saved_tensors
        nb, bw, cwdt, cbdt, wdt, fused = ctx.meta
        R = xy.shape[-1] // 2
        M = xc.numel() // R
        with torch.autocast("cuda", enabled=False):
            xb, y = xy[..., :R], xy[..., R:]
            dxy = torch.empty_like(xy)
            dxc, dgx, dga, dlam, dgb = scan_gelu_bwd_into(xc, gx, ga, lam, gate_bias, h, y, dout, dxy[..., R:])
            if fused:  # d xc (scan) += d gx Wx^T + d ga Wa^T in place, and both weight gradients
                dwx, dwa = gates_bwd_into(xc.view(M, R), dgx.view(M, R), dga.view(M, R), wxc, dxc.view(M, R), bw)
            else:
                dwx, dwa = gates_bmm_bwd_into(xc.view(M, R), dgx.view(M, R), dga.view(M, R), wxc, wac, dxc.view(M, R))
            dcw, dcb = conv1d_bwd_into(dxc, xb, conv_w, dxy[..., :R])
        return dxy, dcw.to(cwdt), dcb.to(cbdt), dwx.to(wdt), dwa.to(wdt), dgb, dlam


def recurrent_core(xy, conv_w, conv_b, wx, wa, gate_bias, lam):
    """(gelu(y) * h, h) from the input projection xy = [x_b | y] of the recurrent block; conv taps/bias,
    Lambda and gate_bias [2, R] in fp32, gate weights [nb, bw, bw]."""
    return _RecurrentCore.apply(xy, conv_w, conv_b, wx, wa, gate_bias, lam)


# ---------------------------------------------------------------------------------------------
# residual add fused into the norm that follows it
# ---------------------------------------------------------------------------------------------
@torch.library.custom_op("hawk_b200::add_rms_norm_fwd", mutates_args=())
def add_rms_norm_fwd(res: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float,
                     out_dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(res + delta, rms_norm(res + delta) * w, rstd); delta must have dtype out_dtype."""
    lib = _lib.load()
    res, delta, w = res.contiguous(), delta.contiguous(), w.contiguous()
    H = res.shape[-1]
    M = res.numel() // H
    new_res = torch.empty_like(res)
    y = torch.empty(res.shape, dtype=out_dtype, device=res.device)
    rstd = torch.empty(M, dtype=torch.float32, device=res.device)
    with _on(res, "add_rms_norm_fwd", 1):
        _lib.check(lib.hawk_add_rms_norm_fwd(res.data_ptr(), delta.data_ptr(), new_res.data_ptr(), w.data_ptr(),
                                             y.data_ptr(), rstd.data_ptr(), M, H, eps, _dt(res), _DT[out_dtype],
                                             _stream(res)), "hawk_add_rms_norm_fwd")
    return new_res, y, rstd


@add_rms_norm_fwd.register_fake
def _(res, delta, w, eps, out_dtype):
    return (torch.empty_like(res, memory_format=torch.contiguous_format), res.new_empty(res.shape, dtype=out_dtype),
            res.new_empty(res.numel() // res.shape[-1], dtype=torch.float32))


@torch.library.custom_op("hawk_b200::add_rms_norm_bwd", mutates_args=())
def add_rms_norm_bwd(gres: Optional[torch.Tensor], dy: torch.Tensor, x_sum: torch.Tensor, w: torch.Tensor,
                     rstd: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(d res, d delta, d w): d res = gres + norm-backward(dy); d delta is the same in dy's dtype."""
    lib = _lib.load()
    dy, x_sum, w = dy.contiguous(), x_sum.contiguous(), w.contiguous()
    if gres is not None:
        gres = gres.contiguous()
    H = x_sum.shape[-1]
    M = x_sum.numel() // H
    dx = torch.empty_like(x_sum)
    ddelta = torch.empty(x_sum.shape, dtype=dy.dtype, device=x_sum.device)
    dw = torch.empty(H, dtype=torch.float32, device=x_sum.device)
    ws_bytes = lib.hawk_rms_norm_bwd_workspace_bytes(H)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x_sum.device)
    with _on(x_sum, "add_rms_norm_bwd", 2):
        _lib.check(lib.hawk_add_rms_norm_bwd(dy.data_ptr(), x_sum.data_ptr(), w.data_ptr(), rstd.data_ptr(), _ptr(gres),
                                             dx.data_ptr(), ddelta.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws_bytes,
                                             M, H, _dt(x_sum), _dt(dy), _stream(x_sum)), "hawk_add_rms_norm_bwd")
    return dx, ddelta, dw


@add_rms_norm_bwd.register_fake
def _(gres, dy, x_sum, w, rstd):
    return (torch.empty_like(x_sum), x_sum.new_empty(x_sum.shape, dtype=dy.dtype),
            w.new_empty(w.shape, dtype=torch.float32))


def _arn_setup(ctx, inputs, output):
    _, delta, w, _, _ = inputs
    new_res, _, rstd = output
    ctx.save_for_backward(new_res, w, rstd)
    ctx.w_dtype, ctx.delta_dtype = w.dtype, delta.dtype
    ctx.set_materialize_grads(False)


def _arn_backward(ctx, g_res, g_y, g_rstd):
    new_res, w, rstd = ctx.saved_tensors
    if g_y is None:  # the norm output was not used: only the residual path carries gradient
        if g_res is None:
            return None, None, None, None, None
        return g_res, g_res.to(ctx.delta_dtype), None, None, None
    dx, ddelta, dw = add_rms_norm_bwd(g_res, g_y, new_res, w, rstd)
    return dx, ddelta, dw.to(ctx.w_dtype), None, None


add_rms_norm_fwd.register_autograd(_arn_backward, setup_context=_arn_setup)


def add_rms_norm(res, delta, weight, eps: float = 1e-6, out_dtype=None):
    """(res + delta, rms_norm(res + delta) * weight): the block's residual add and the norm after it in
    one pass each way.  `delta` None means a plain norm of `res`."""
    out_dtype = out_dtype or res.dtype
    w32 = weight if weight.dtype == torch.float32 else weight.float()
    if delta is None:
        return res, rms_norm_fwd(res, w32, eps, out_dtype)[0]
    if delta.dtype != out_dtype:
        delta = delta.to(out_dtype)
    new_res, y, _ = add_rms_norm_fwd(res, delta, w32, eps, out_dtype)
    return new_res, y
