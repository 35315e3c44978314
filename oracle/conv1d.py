"""CPU oracle for the width-W causal depthwise temporal convolution.

TEST INFRASTRUCTURE ONLY (see oracle/scan.py for the rule).

Restates hawk/external.py:49-95 (Conv1D.doc_mask_forward with prompt_len = 0):
for temporal_shift k = 0..W-1 the window x[:, 0:T-k] is left-padded with k zero
rows (external.py:100-136) and multiplied by w[W-1-k] (external.py:88-90); the
bias is added last (external.py:93).  Hence

    y[b,t,d] = b[d] + sum_{k=0}^{W-1} w[W-1-k, d] * x[b, t-k, d],   x[b, t<0] = 0.

Pinned by tests/golden/conv1d_ref.npz (the reference module itself, run on CPU).
"""
from __future__ import annotations

import torch


def conv1d_fwd(x, w, b, *, compute=torch.float32):
    """x [B,T,D] (any strides), w [W,D], b [D] -> y [B,T,D] in `compute`."""
    x = x.to(compute)
    w = w.to(compute)
    b = b.to(compute)
    B, T, D = x.shape
    W = w.shape[0]
    y = torch.zeros(B, T, D, dtype=compute)
    for k in range(min(W, T)):  # external.py:73 "valid" clamp
        y[:, k:] += x[:, : T - k] * w[W - 1 - k][None, None, :]
    y += b[None, None]
    return y


def conv1d_bwd(x, w, go, *, compute=torch.float32):
    """Gradients of conv1d_fwd: (dx [B,T,D], dw [W,D], db [D])."""
    x = x.to(compute)
    w = w.to(compute)
    go = go.to(compute)
    B, T, D = x.shape
    W = w.shape[0]
    dx = torch.zeros(B, T, D, dtype=compute)
    dw = torch.zeros(W, D, dtype=compute)
    for k in range(min(W, T)):
        # y[t] += w[W-1-k] x[t-k]  =>  dx[s] += w[W-1-k] go[s+k];  dw[W-1-k] += sum go[t] x[t-k]
        dx[:, : T - k] += go[:, k:] * w[W - 1 - k][None, None, :]
        dw[W - 1 - k] = (go[:, k:] * x[:, : T - k]).sum(dim=(0, 1))
    db = go.sum(dim=(0, 1))
    return dx, dw, db
