"""CPU oracle for the fused linear + cross-entropy op.

TEST INFRASTRUCTURE ONLY (see oracle/scan.py for the rule).

Restates hawk/fused_cross_entropy.py:13-64 (CrossEntropyLoopedFused.forward):
rows are processed in chunks of 2048 (:18-20); per chunk
logits = act @ W^T (:28), a max-shifted softmax (:31-34), the summed loss
max + log(sum exp) - correct_logit (:37-44), dprobs = probs - onehot (:47-52),
dW += dprobs^T @ act (:55), dact = dprobs @ W (:56); both gradients and the loss
are scaled by 1/N at the end (:59-64).  backward multiplies the stored gradients
by the scalar upstream gradient (:66-73).

`autocast_bf16=True` emulates what torch.autocast(bfloat16) does to this code on a
GPU: the three matmuls take bf16-rounded operands, accumulate in fp32 and round
their result to bf16; exp/sum/log run in fp32.

Pinned by tests/golden/linear_ce_ref.npz (the reference Function run eagerly on
CPU in fp32).
"""
from __future__ import annotations

import torch

CHUNK = 2048  # hawk/fused_cross_entropy.py:18


def _mm(a, b, bf16):
    if not bf16:
        return a @ b
    a = a.to(torch.bfloat16).to(torch.float32)
    b = b.to(torch.bfloat16).to(torch.float32)
    return (a @ b).to(torch.bfloat16).to(torch.float32)


def linear_ce_fwd_bwd(weight, act, labels, *, compute=torch.float32, autocast_bf16=False, chunk=CHUNK):
    """weight [V,H], act [N,H], labels [N] int64 -> (loss 0-dim, dW [V,H], dact [N,H])."""
    weight = weight.to(compute)
    act = act.to(compute)
    N = act.shape[0]
    dW = torch.zeros_like(weight)
    dact = torch.empty_like(act)
    loss = torch.zeros((), dtype=compute)
    for s in range(0, N, chunk):
        e = min(s + chunk, N)
        a = act[s:e]
        lab = labels[s:e]
        logits = _mm(a, weight.T, autocast_bf16)
        mx = logits.max(dim=-1, keepdim=True)[0]
        ex = torch.exp(logits - mx)
        se = ex.sum(dim=-1, keepdim=True)
        probs = ex / se
        correct = logits.gather(1, lab[:, None])
        loss = loss + (mx.squeeze(-1) + torch.log(se.squeeze(-1)) - correct.squeeze(-1)).sum()
        dprobs = probs.clone()
        dprobs.scatter_(1, lab[:, None], dprobs.gather(1, lab[:, None]) - 1)
        dW += _mm(dprobs.T, a, autocast_bf16)
        dact[s:e] = _mm(dprobs, weight, autocast_bf16)
    scale = 1.0 / N
    return scale * loss, dW * scale, dact * scale


def linear_ce_direct(weight, act, labels, *, compute=torch.float64):
    """Independent check: autograd through F.cross_entropy(act @ W^T)."""
    w = weight.detach().to(compute).requires_grad_(True)
    a = act.detach().to(compute).requires_grad_(True)
    loss = torch.nn.functional.cross_entropy(a @ w.T, labels)
    dw, da = torch.autograd.grad(loss, (w, a))
    return loss.detach(), dw, da
