"""CPU oracle for the RG-LRU scan (forward and backward).

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file; it
is the checker that tests, the smoke run and the CPU-baseline leg of the bench
compare the CUDA kernels against.

The reference ships the scan only as two Triton kernels, so this is a
restatement of their arithmetic in plain torch on CPU, vectorised over
(batch, channel) and sequential over time:

  forward   hawk/scan_fused.py:44-109   (sequential_scan_fwd_kernel)
  backward  hawk/scan_fused.py:123-317  (sequential_scan_bwd_kernel)
  helpers   hawk/scan_fused.py:10-30    (clipped_sqrt_grad, softplus_fwd/bwd, sigmoid_bwd)
  batch sum hawk/scan_fused.py:424      (a_param_batched.sum(0))

Operation order follows the reference expression by expression so that, with the
reference's own rounding points emulated (`store="bf16_trunc"` is what the Triton
interpreter does on CPU, `store="bf16_rne"` what a GPU does), the result is
bit-identical to the reference kernels.  Pinned by tests/golden/scan_triton_interp.npz,
which was produced by running the unmodified reference kernels under the Triton
interpreter (tests/golden/make_golden.py).

`store=None` keeps every value in the compute dtype; that is the form the CUDA
kernels are held to (1e-5 in fp32), since they store in the tensor's own dtype.
"""
from __future__ import annotations

import torch

C_GATE = -8.0  # hawk/scan_fused.py:44,123
MAX_SQRT_GRADIENT = 1000.0  # hawk/scan_fused.py:11


def _store_fn(store):
    if store is None:
        return lambda t: t
    if store == "bf16_rne":
        return lambda t: t.to(torch.bfloat16).to(t.dtype)
    if store == "bf16_trunc":

        def trunc(t):
            assert t.dtype == torch.float32
            return (t.contiguous().view(torch.int32) & -65536).view(torch.float32)

        return trunc
    raise ValueError(f"unknown store mode {store!r}")


def softplus_fwd(lam):
    """hawk/scan_fused.py:18-20 (naive form, no threshold)."""
    return torch.log(1 + torch.exp(lam))


def softplus_bwd(lam):
    """hawk/scan_fused.py:23-25."""
    return torch.exp(lam) / (1 + torch.exp(lam))


def clipped_sqrt_grad(v):
    """hawk/scan_fused.py:10-15: 1/sqrt(max(4 v, 1e-6))."""
    min_value = 1.0 / (MAX_SQRT_GRADIENT * MAX_SQRT_GRADIENT)
    scaled = 4.0 * v
    clipped = torch.where(scaled > min_value, scaled, torch.full_like(scaled, min_value))
    return 1.0 / torch.sqrt(clipped)


def _gates(x, gx, ga, lam, compute):
    """Per-element quantities shared by forward and backward (scan_fused.py:63-105)."""
    x = x.to(compute)
    gx = gx.to(compute)
    ga = ga.to(compute)
    lam = lam.to(compute)
    sp = softplus_fwd(lam)
    i = torch.sigmoid(gx)
    r = torch.sigmoid(ga)
    log_a = C_GATE * r * sp
    a = torch.exp(log_a)
    a2 = torch.exp(2 * log_a)
    m = torch.sqrt(1 - a2)
    return x, gx, ga, lam, sp, i, r, log_a, a, a2, m


def rglru_scan_fwd(x, gx, ga, lam, *, compute=torch.float32, store=None, h0=None):
    """h[b,t,d] of the RG-LRU recurrence; h_{-1} = h0 (zero in the reference).

    x, gx, ga: [B,T,D]; lam: [D].  Returns h in the compute dtype (values rounded
    through `store` exactly where the reference rounds its stores; the carried
    state itself is never rounded, scan_fused.py:79,107).
    """
    st = _store_fn(store)
    x, gx, ga, lam, sp, i, r, log_a, a, a2, m = _gates(x, gx, ga, lam, compute)
    beta = (x * i) * m  # gated_x * multiplier, :103-105
    B, T, D = x.shape
    h = torch.empty_like(beta)
    if h0 is None:
        state = beta[:, 0]  # :79  (a_0 unused)
    else:
        state = a[:, 0] * h0.to(compute) + beta[:, 0]
    h[:, 0] = st(state)
    for t in range(1, T):
        state = a[:, t] * state + beta[:, t]  # :107
        h[:, t] = st(state)
    return h


def rglru_scan_bwd(x, gx, ga, lam, h_saved, go, *, compute=torch.float32, store=None):
    """(dx, dgx, dga, dlam) of the reference backward kernel.

    h_saved is the forward OUTPUT as stored (the reference re-reads the rounded h,
    scan_fused.py:133,154,218); go is the upstream gradient of h.
    dlam is accumulated in the compute dtype per batch row and then summed over
    the batch (scan_fused.py:130,317,424).
    """
    st = _store_fn(store)
    x, gx, ga, lam, sp, i, r, log_a, a, a2, m = _gates(x, gx, ga, lam, compute)
    go = go.to(compute)
    h_saved = h_saved.to(compute)
    B, T, D = x.shape

    # dh_t = go_t + a_{t+1} dh_{t+1}  (:153, :213-219, :273-276)
    dh = torch.empty_like(go)
    g = go[:, T - 1]
    dh[:, T - 1] = g
    for t in range(T - 2, -1, -1):
        g = a[:, t + 1] * g
        g = g + go[:, t]
        dh[:, t] = g

    hprev = torch.zeros_like(h_saved)
    hprev[:, 1:] = h_saved[:, :-1]

    d_alpha = dh * hprev
    sg = clipped_sqrt_grad(1 - a2)
    extra = -2.0 * a2
    second = dh * (i * x) * sg * extra
    dlog_a = d_alpha * a
    dlog_a = dlog_a + second
    dlog_a[:, 0] = second[:, 0]  # t = 0 has no d_alpha term (:303-307)

    sig_bwd_a = r * (1 - r)
    sig_bwd_x = i * (1 - i)
    dga = sig_bwd_a * dlog_a * C_GATE * sp
    dx = dh * m * i
    dgx = dh * m * x * sig_bwd_x
    contrib = dlog_a * C_GATE * r * softplus_bwd(lam)
    # sequential accumulation over t from T-1 down to 0, as the kernel does
    acc = torch.zeros(B, D, dtype=compute)
    for t in range(T - 1, -1, -1):
        acc = acc + contrib[:, t]
    dlam = acc.sum(dim=0)
    return st(dx), st(dgx), st(dga), dlam


def rglru_scan_autograd(x, gx, ga, lam, go, *, compute=torch.float64):
    """Independent check: torch.autograd through a differentiable forward.

    Equals rglru_scan_bwd except where the reference clamps the sqrt gradient
    (1 - a^2 < 2.5e-7) and where it re-reads a rounded h.
    """
    xs = [t.detach().to(compute).requires_grad_(True) for t in (x, gx, ga, lam)]
    x_, gx_, ga_, lam_ = xs
    sp = torch.nn.functional.softplus(lam_)
    i = torch.sigmoid(gx_)
    r = torch.sigmoid(ga_)
    log_a = C_GATE * r * sp
    a = torch.exp(log_a)
    m = torch.sqrt(1 - torch.exp(2 * log_a))
    beta = x_ * i * m
    T = x.shape[1]
    hs = [beta[:, 0]]
    for t in range(1, T):
        hs.append(a[:, t] * hs[-1] + beta[:, t])
    h = torch.stack(hs, dim=1)
    grads = torch.autograd.grad(h, xs, go.to(compute))
    return (h.detach(),) + tuple(grads)


def closed_form_kat(lam, T, *, compute=torch.float64):
    """Known answer for gx = ga = 0, x = 1:  h_t = m (1 - a^(t+1)) / (1 - a)
    with rho = exp(-softplus(lam)), a = rho^4, m = 0.5 sqrt(1 - a^2)."""
    lam = lam.to(compute)
    a = torch.exp(-4.0 * torch.nn.functional.softplus(lam))
    m = 0.5 * torch.sqrt(1 - a * a)
    t = torch.arange(1, T + 1, dtype=compute)[:, None]
    return (m * (1 - a[None, :] ** t) / (1 - a))[None]  # [1,T,D]


def rnn_param_ring(D, *, min_rad=0.9, max_rad=0.999, eps=1e-8, generator=None):
    """Lambda drawn as hawk/external.py:153-168 (rnn_param_init, softplus transform):
    u ~ U[min^2+eps, max^2+eps];  lam = log(exp(-0.5 log u) - 1)."""
    u = torch.empty(D, dtype=torch.float32).uniform_(min_rad**2 + eps, max_rad**2 + eps, generator=generator)
    return torch.log(torch.exp(-0.5 * torch.log(u)) - 1.0)
