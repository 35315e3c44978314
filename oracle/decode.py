"""CPU oracle for the cached single-token decode step of one Hawk block.

TEST INFRASTRUCTURE ONLY (see oracle/scan.py for the rule).

Restates, for an arbitrary batch (the reference cache asserts batch 1,
hawk/cache.py:30-31,38-39):

  conv over the 4-token window [conv_state(3) | x_new]   hawk/hawk.py:168-179
  cache roll                                              hawk/cache.py:37-43
  gate -> (a, normalised x)                               hawk/hawk.py:137-151
  h = a * state + normalised x                            hawk/hawk.py:196
"""
from __future__ import annotations

import torch

from .scan import C_GATE


def conv_step(x_new, conv_state, w, b, *, compute=torch.float32):
    """x_new [B,D], conv_state [B,W-1,D] (oldest first), w [W,D], b [D].

    Returns (y [B,D], new_conv_state [B,W-1,D]).  y is the last row of the
    reference's conv over the concatenated window (hawk.py:169,176-179):
    y = b + w[W-1] x_new + sum_{j<W-1} w[j] conv_state[:, j].
    """
    W = w.shape[0]
    window = torch.cat([conv_state.to(compute), x_new.to(compute)[:, None]], dim=1)  # [B,W,D]
    y = (window * w.to(compute)[None]).sum(dim=1) + b.to(compute)[None]
    new_state = window[:, 1:].clone()  # roll(-1) then overwrite last (cache.py:42-43)
    assert new_state.shape[1] == W - 1
    return y, new_state


def rglru_step(x, gx, ga, lam, state, *, compute=torch.float32):
    """One recurrence step.  x, gx, ga, state: [B,D]; lam [D].  Returns h [B,D]."""
    x = x.to(compute)
    i = torch.sigmoid(gx.to(compute))
    r = torch.sigmoid(ga.to(compute))
    log_a = C_GATE * r * torch.nn.functional.softplus(lam.to(compute))
    a = torch.exp(log_a)
    a2 = torch.exp(2 * log_a)
    m = torch.sqrt(1 - a2)
    return a * state.to(compute) + (x * i) * m
