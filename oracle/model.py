"""CPU oracle for the Hawk block and model around the hot-path ops.

TEST INFRASTRUCTURE ONLY (see oracle/scan.py for the rule).

A functional restatement of hawk/hawk.py driven by a reference-format state dict
(keys as produced by HawkModel.state_dict(): `embed_tokens.weight`,
`layers.{i}.recc.{rg_lru_a_param, input_xy.weight, rg_lru_input_gate.{w,b},
rg_lru_a_gate.{w,b}, resid_proj.weight, conv1d.{w,b}}`,
`layers.{i}.mlp.{gate_up_proj,resid_proj}.weight`,
`layers.{i}.{input_norm,post_recurrent_norm}.weight`, `norm.weight`,
`lm_head.weight`).  Everything is differentiable torch on CPU, so gradients come
from autograd; the scan inside is the differentiable statement of
oracle/scan.py's forward.

Pinned by tests/golden/model_ref.npz (the reference HawkModel itself on CPU in
fp32 with its Triton scan rebound to oracle.scan, see tests/golden/make_golden.py).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .scan import C_GATE

EPS = 1e-6  # hawk/hawk.py:48


def rms_norm(x, weight):
    """hawk/hawk.py:53-58."""
    xf = x.float()
    out = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + EPS)).type_as(x)
    return out * weight


def block_diag_linear(x, w, b):
    """hawk/external.py:224-233: x [...,(h i)] , w [h,i,j], b [h,j]."""
    nb, bw, _ = w.shape
    xs = x.reshape(*x.shape[:-1], nb, bw)
    y = torch.einsum("...hi,hij->...hj", xs, w) + b
    return y.reshape(*x.shape)


def conv1d(x, w, b):
    """hawk/external.py:49-95 (differentiable form of oracle/conv1d.py)."""
    T = x.shape[1]
    W = w.shape[0]
    y = 0.0
    for k in range(min(W, T)):
        win = F.pad(x[:, : T - k], (0, 0, k, 0))
        y = y + win * w[W - 1 - k][None, None, :]
    return y + b[None, None]


def scan(x, gx, ga, lam):
    """Differentiable forward of hawk/scan_fused.py:57-109 (h_{-1} = 0)."""
    sp = torch.log(1 + torch.exp(lam))
    i = torch.sigmoid(gx)
    r = torch.sigmoid(ga)
    log_a = C_GATE * r * sp
    a = torch.exp(log_a)
    m = torch.sqrt(1 - torch.exp(2 * log_a))
    beta = (x * i) * m
    hs = [beta[:, 0]]
    for t in range(1, x.shape[1]):
        hs.append(a[:, t] * hs[-1] + beta[:, t])
    return torch.stack(hs, dim=1)


def hawk_block(sd, prefix, x, *, taps=None):
    """Training branch of Hawk.forward, hawk/hawk.py:153-203."""
    p = lambda k: sd[prefix + k]
    xy = F.linear(x, p("input_xy.weight"))
    xb, yb = torch.chunk(xy, 2, dim=-1)
    xc = conv1d(xb, p("conv1d.w"), p("conv1d.b"))
    gx = block_diag_linear(xc, p("rg_lru_input_gate.w"), p("rg_lru_input_gate.b"))
    ga = block_diag_linear(xc, p("rg_lru_a_gate.w"), p("rg_lru_a_gate.b"))
    h = scan(xc, gx, ga, p("rg_lru_a_param").float())
    if taps is not None:
        taps.update(conv_out=xc, gx=gx, ga=ga, h=h)
    return F.linear(F.gelu(yb) * h, p("resid_proj.weight"))


def mlp(sd, prefix, x):
    """hawk/hawk.py:81-86."""
    gu = F.linear(x, sd[prefix + "gate_up_proj.weight"])
    gate, up = torch.chunk(gu, 2, dim=-1)
    return F.linear(F.gelu(gate) * up, sd[prefix + "resid_proj.weight"])


def layer(sd, i, x):
    """RNNLayer.forward, hawk/hawk.py:218-236."""
    pre = f"layers.{i}."
    x = x + hawk_block(sd, pre + "recc.", rms_norm(x, sd[pre + "input_norm.weight"]))
    x = x + mlp(sd, pre + "mlp.", rms_norm(x, sd[pre + "post_recurrent_norm.weight"]))
    return x


def num_layers(sd):
    return 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("layers."))


def hidden_states(sd, input_ids):
    """hawk/hawk.py:271-284."""
    x = F.embedding(input_ids, sd["embed_tokens.weight"])
    for i in range(num_layers(sd)):
        x = layer(sd, i, x)
    return rms_norm(x, sd["norm.weight"])


def logits(sd, input_ids):
    """hawk/hawk.py:302-303."""
    return F.linear(hidden_states(sd, input_ids), sd["lm_head.weight"])


def loss(sd, input_ids, labels):
    """Labels branch, hawk/hawk.py:291-300: next-token shift then mean cross-entropy."""
    hs = hidden_states(sd, input_ids)
    shift_x = hs[..., :-1, :].reshape(-1, hs.shape[-1])
    shift_labels = labels[..., 1:].reshape(-1)
    return F.cross_entropy(F.linear(shift_x, sd["lm_head.weight"]), shift_labels)


def dezero(sd, seed):
    """Re-draw the zero-initialised families (lm_head and both resid_proj per layer,
    hawk/hawk.py:79,128,258) with LeCun normal from a seeded generator, so that the
    scan and the conv influence the loss at step 0."""
    g = torch.Generator().manual_seed(seed)
    out = dict(sd)
    for k in sorted(sd):
        if k == "lm_head.weight" or k.endswith("resid_proj.weight"):
            w = sd[k]
            out[k] = torch.randn(w.shape, generator=g, dtype=w.dtype) / (w.shape[1] ** 0.5)
    return out


# ---------------------------------------------------------------------------
# cached decode (HawkModel(use_cache=True)), generalised to any batch size
# ---------------------------------------------------------------------------
from . import decode as _dec  # noqa: E402


def prefill(sd, input_ids, *, state_dtype=torch.bfloat16):
    """First call with empty caches (hawk/hawk.py:172-174,186-190,286-288).

    Returns (logits [B,T,V], caches) where caches[i] = dict(recc=[B,R] in
    `state_dtype` (the reference cache is bf16, hawk/cache.py:15), conv=[B,3,R]).
    """
    caches = []
    x = F.embedding(input_ids, sd["embed_tokens.weight"])
    for i in range(num_layers(sd)):
        pre = f"layers.{i}."
        taps = {}
        xin = rms_norm(x, sd[pre + "input_norm.weight"])
        xb = torch.chunk(F.linear(xin, sd[pre + "recc.input_xy.weight"]), 2, dim=-1)[0]
        x = x + hawk_block(sd, pre + "recc.", xin, taps=taps)
        x = x + mlp(sd, pre + "mlp.", rms_norm(x, sd[pre + "post_recurrent_norm.weight"]))
        caches.append(dict(recc=taps["h"][:, -1].to(state_dtype), conv=xb[:, -3:].clone()))
    return F.linear(rms_norm(x, sd["norm.weight"]), sd["lm_head.weight"]), caches


def decode_step(sd, token_ids, caches, *, state_dtype=torch.bfloat16):
    """One cached token (hawk/hawk.py:168-170,176-182,193-199).  token_ids [B,1]."""
    x = F.embedding(token_ids, sd["embed_tokens.weight"])[:, 0]  # [B,H]
    new_caches = []
    for i, c in enumerate(caches):
        pre = f"layers.{i}."
        p = lambda k: sd[pre + "recc." + k]
        xin = rms_norm(x, sd[pre + "input_norm.weight"])
        xb, yb = torch.chunk(F.linear(xin, p("input_xy.weight")), 2, dim=-1)
        xc, conv_state = _dec.conv_step(xb, c["conv"], p("conv1d.w"), p("conv1d.b"))
        gx = block_diag_linear(xc, p("rg_lru_input_gate.w"), p("rg_lru_input_gate.b"))
        ga = block_diag_linear(xc, p("rg_lru_a_gate.w"), p("rg_lru_a_gate.b"))
        h = _dec.rglru_step(xc, gx, ga, p("rg_lru_a_param"), c["recc"])
        x = x + F.linear(F.gelu(yb) * h, p("resid_proj.weight"))
        x = x + mlp(sd, pre + "mlp.", rms_norm(x, sd[pre + "post_recurrent_norm.weight"]))
        new_caches.append(dict(recc=h.to(state_dtype), conv=conv_state))
    logits = F.linear(rms_norm(x, sd["norm.weight"]), sd["lm_head.weight"])
    return logits[:, None], new_caches


def random_state_dict(vocab, hidden, intermediate, layers, recurrent, num_blocks, conv_width, *, seed=0):
    """A reference-format state dict drawn with the reference's initialisation families
    (hawk/hawk.py:77-79,124-132,256-258; hawk/external.py:45-47,153-168,214-222): LeCun normal for the
    embedding, input_xy and gate_up_proj; zeros for lm_head and both resid_proj; ring init for Lambda;
    N(0, 0.01/width) conv taps; N(0, 1/bw) gate blocks; zero biases; unit norm weights."""
    from .scan import rnn_param_ring
    g = torch.Generator().manual_seed(seed)
    n = lambda *shape, std: torch.randn(*shape, generator=g) * std
    bw = recurrent // num_blocks
    sd = {"embed_tokens.weight": n(vocab, hidden, std=hidden ** -0.5), "norm.weight": torch.ones(hidden),
          "lm_head.weight": torch.zeros(vocab, hidden)}
    for i in range(layers):
        p = f"layers.{i}."
        sd[p + "recc.rg_lru_a_param"] = rnn_param_ring(recurrent, generator=g)
        sd[p + "recc.input_xy.weight"] = n(2 * recurrent, hidden, std=hidden ** -0.5)
        for gate in ("rg_lru_input_gate", "rg_lru_a_gate"):
            sd[p + f"recc.{gate}.w"] = n(num_blocks, bw, bw, std=bw ** -0.5)
            sd[p + f"recc.{gate}.b"] = torch.zeros(num_blocks, bw)
        sd[p + "recc.resid_proj.weight"] = torch.zeros(hidden, recurrent)
        sd[p + "recc.conv1d.w"] = n(conv_width, recurrent, std=(0.01 / conv_width) ** 0.5)
        sd[p + "recc.conv1d.b"] = torch.zeros(recurrent)
        sd[p + "mlp.gate_up_proj.weight"] = n(2 * intermediate, hidden, std=hidden ** -0.5)
        sd[p + "mlp.resid_proj.weight"] = torch.zeros(hidden, intermediate)
        sd[p + "input_norm.weight"] = torch.ones(hidden)
        sd[p + "post_recurrent_norm.weight"] = torch.ones(hidden)
    return sd
