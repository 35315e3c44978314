"""Hawk model shell around the sm_100a operators.

Mirrors the reference's public interface (hawk/hawk.py, hawk/cache.py, hawk/external.py):
`HawkConfig` (same seven fields), `HawkModel(config, use_cache=False)` with
`forward(input_ids, labels=None, layer_past=None)` returning the loss, the logits, or
`(logits, caches)`; module and parameter names are the reference's, so state dicts interchange
(`embed_tokens.weight`, `layers.{i}.recc.{rg_lru_a_param, input_xy.weight, rg_lru_input_gate.{w,b},
rg_lru_a_gate.{w,b}, resid_proj.weight, conv1d.{w,b}}`, `layers.{i}.mlp.{gate_up_proj,resid_proj}.weight`,
`layers.{i}.{input_norm,post_recurrent_norm}.weight`, `norm.weight`, `lm_head.weight`).

The recurrent block calls hawk_b200.ops for the temporal conv, the RG-LRU scan, the fused linear
cross-entropy and the cached decode step; dense projections stay on cuBLAS through torch.
Differences from the reference, all inside its bf16-autocast tolerance:
  * the conv writes the activation dtype directly (the reference promotes to fp32 and the scan's
    autocast wrapper rounds back to bf16, hawk/external.py:88-93, hawk/scan_fused.py:428);
  * Lambda stays fp32 inside the scan;
  * the decode cache holds any batch size (the reference asserts batch 1, hawk/cache.py:30-31).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops


@dataclass
class HawkConfig:
    """hawk/hawk.py:21-29."""
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    recurrent_size: int
    num_blocks: int
    conv_width: int


def _lecun_normal_(w: torch.Tensor, fan_in: int) -> None:
    nn.init.normal_(w, mean=0.0, std=1.0 / math.sqrt(fan_in))  # hawk/hawk.py:37-39


def ring_init_(lam: torch.Tensor, min_rad: float = 0.9, max_rad: float = 0.999, eps: float = 1e-8) -> torch.Tensor:
    """Lambda with exp(-softplus(Lambda)) uniform on [min_rad, max_rad] in squared radius
    (hawk/external.py:153-168): Lambda = log(u^(-1/2) - 1), u ~ U[min^2 + eps, max^2 + eps]."""
    with torch.no_grad():
        lam.uniform_(min_rad**2 + eps, max_rad**2 + eps)
        lam.copy_(torch.log(torch.rsqrt(lam) - 1.0))
    return lam


def rnn_param_init(tensor: torch.Tensor, min_rad: float, max_rad: float, transform: str = "softplus",
                   eps: float = 1e-8) -> torch.Tensor:
    """The reference's name and signature for the ring initialisation (hawk/external.py:153-168)."""
    if transform != "softplus":
        raise NotImplementedError()  # as the reference
    return ring_init_(tensor, min_rad, max_rad, eps)


def lecun_init(w: torch.Tensor, d_in: int) -> None:
    """The reference's name for the N(0, 1/sqrt(d_in)) initialisation (hawk/hawk.py:37-39)."""
    _lecun_normal_(w, d_in)


class RMSNorm(nn.Module):
    """hawk/hawk.py:47-58: statistics in fp32, result in the input dtype, times the weight."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    @staticmethod
    def _out_dtype(x):
        # under autocast the only consumer is a Linear, which would round its input to bf16 anyway
        return torch.bfloat16 if (x.is_cuda and torch.is_autocast_enabled("cuda")) else None

    def _weight32(self):
        """The kernels take the weight in fp32.  A model converted to bf16 for inference would otherwise pay a
        cast launch per norm per token (49 of a decode step's 244 launches): keep an fp32 copy, remade when
        the weight is written (version counter) or replaced."""
        w = self.weight
        if w.dtype == torch.float32:
            return w
        if w.requires_grad and torch.is_grad_enabled():
            return w.float()  # training a reduced-precision weight: keep the cast in the autograd graph
        key = (w.data_ptr(), w._version, w.device)
        if getattr(self, "_w32_key", None) != key:
            self._w32 = w.detach().float()
            self._w32_key = key
        return self._w32

    def forward(self, x):
        return ops.rms_norm(x, self._weight32(), self.eps, out_dtype=self._out_dtype(x))

    def add_forward(self, residual, delta):
        """(residual + delta, norm(residual + delta)); delta None = plain norm.  The residual add that
        precedes every norm (hawk/hawk.py:229,234) is fused into it."""
        return ops.add_rms_norm(residual, delta, self._weight32(), self.eps, out_dtype=self._out_dtype(residual))


class BlockDiagonalLinear(nn.Module):
    """`num_blocks` independent [bw, bw] projections plus bias (hawk/external.py:171-233).
    One strided-batch GEMM with the bias folded in; parameters `w` [nb, bw, bw], `b` [nb, bw]."""

    def __init__(self, width: int, num_blocks: int, w_init_variance_scale: float = 1.0):
        super().__init__()
        self.width, self.num_blocks = width, num_blocks
        self.block_width = width // num_blocks
        self.w = nn.Parameter(torch.empty(num_blocks, self.block_width, self.block_width))
        self.b = nn.Parameter(torch.zeros(num_blocks, self.block_width))
        nn.init.normal_(self.w, mean=0.0, std=math.sqrt(w_init_variance_scale / self.block_width))

    def forward(self, x):
        lead = x.shape[:-1]
        xb = x.reshape(-1, self.num_blocks, self.block_width).transpose(0, 1)  # [nb, M, bw]
        y = torch.baddbmm(self.b.unsqueeze(1), xb, self.w)                      # [nb, M, bw]
        return y.transpose(0, 1).reshape(*lead, self.width)


class RNNCache:
    """Decode state of one recurrent block (hawk/cache.py:4-46), for any batch size:
    `recc_state` [B,1,D] and `conv_state` [B,W-1,D] (oldest row first), bf16 like the reference."""

    def __init__(self, state_dim: int, device, temporal_conv_width: int = 4, batch_size: int = 1,
                 dtype: torch.dtype = torch.bfloat16):
        self.state_dim = state_dim
        self.device = torch.device(device)
        self.temporal_conv_width = temporal_conv_width
        self.conv_cache_size = temporal_conv_width - 1
        self.current_cache_size = 0
        self.recc_state = torch.full((batch_size, 1, state_dim), float("nan"), dtype=dtype, device=device)
        self.conv_state = torch.full((batch_size, self.conv_cache_size, state_dim), float("nan"), dtype=dtype,
                                     device=device)

    def update_cache(self, new_state: torch.Tensor) -> None:
        assert new_state.shape == self.recc_state.shape, (new_state.shape, self.recc_state.shape)
        self.recc_state.copy_(new_state)
        self.current_cache_size = 1

    def update_conv_cache(self, new_state: torch.Tensor) -> None:
        assert new_state.shape[0] == self.conv_state.shape[0] and new_state.shape[1] == 1
        self.conv_state = torch.cat([self.conv_state[:, 1:], new_state.to(self.conv_state.dtype)], dim=1)

    def __repr__(self) -> str:
        return (f"RNNCache(batch={self.recc_state.shape[0]}, state_dim={self.state_dim}, "
                f"filled={self.current_cache_size}, conv_width={self.temporal_conv_width})")


class Linear(nn.Linear):
    """nn.Linear without bias (same parameter name and state-dict key) whose forward goes through
    `ops.linear`: under CUDA bf16 autocast the weight cast and the weight-gradient cast are fused away.

    The bf16 copy an optimiser leaves here is trusted while `weight._version` is the version it was written
    for.  Every in-place operation on the parameter, `load_state_dict` and `.to()` change the version (or the
    tensor) and so fall back to a fresh cast; a write through `weight.data` (e.g. `weight.data.copy_(w)`) does
    NOT change the version: after such a write call `drop_bf16_copy()` (or `drop_bf16_copies(model)`)."""

    # bf16 copy of the weight kept current by an optimiser that updates both in one pass
    # (train.FusedAdamW); valid only while the fp32 weight still has the version it was written for
    weight_bf16: Optional[torch.Tensor] = None
    weight_bf16_version: int = -1

    def drop_bf16_copy(self) -> None:
        self.weight_bf16, self.weight_bf16_version = None, -1

    def forward(self, x):
        if self.bias is not None:
            return super().forward(x)
        wb = self.weight_bf16
        if wb is not None and (torch.compiler.is_compiling() or self.weight_bf16_version != self.weight._version
                               or wb.device != self.weight.device):
            wb = None  # stale, or traced code (which must not depend on a tensor's version): cast instead
        return ops.linear(x, self.weight, wb)


def drop_bf16_copies(module: nn.Module) -> None:
    """Forget the optimiser-written bf16 weight copies of every `Linear` under `module` (needed only after
    writing weights behind autograd's back, see `Linear`)."""
    for m in module.modules():
        if isinstance(m, Linear):
            m.drop_bf16_copy()


class MLP(nn.Module):
    """Gated GELU feed-forward (hawk/hawk.py:61-86); `resid_proj` starts at zero."""

    def __init__(self, config: HawkConfig):
        super().__init__()
        self.gate_up_proj = Linear(config.hidden_size, 2 * config.intermediate_size, bias=False)
        self.resid_proj = Linear(config.intermediate_size, config.hidden_size, bias=False)
        _lecun_normal_(self.gate_up_proj.weight, config.hidden_size)
        nn.init.zeros_(self.resid_proj.weight)

    def forward(self, x):
        return self.resid_proj(ops.geglu(self.gate_up_proj(x)))  # gelu(gate) * up in one pass


class Hawk(nn.Module):
    """The recurrent block (hawk/hawk.py:89-203)."""

    def __init__(self, config: HawkConfig, use_cache: bool = False):
        super().__init__()
        self.config = config
        self.use_cache = use_cache
        R = config.recurrent_size
        self.input_xy = Linear(config.hidden_size, 2 * R, bias=False)
        self.rg_lru_input_gate = BlockDiagonalLinear(R, config.num_blocks)
        self.rg_lru_a_gate = BlockDiagonalLinear(R, config.num_blocks)
        self.rg_lru_a_param = nn.Parameter(torch.empty(R, dtype=torch.float32))
        self.resid_proj = Linear(R, config.hidden_size, bias=False)
        self.conv1d = ops.Conv1D(width=R, temporal_width=config.conv_width)
        self._fp32_cache = {}
        ring_init_(self.rg_lru_a_param)
        _lecun_normal_(self.input_xy.weight, config.hidden_size)
        nn.init.zeros_(self.resid_proj.weight)

    def _fp32(self, name: str, p: torch.Tensor) -> torch.Tensor:
        """fp32 view of a small parameter for the kernels that take fp32 taps / Lambda; when the model
        has been cast to bf16 the converted copy is kept until the parameter changes."""
        if p.dtype == torch.float32:
            return p
        hit = self._fp32_cache.get(name)
        if hit is None or hit[0] != p._version or hit[1].device != p.device:
            hit = (p._version, p.detach().float())
            self._fp32_cache[name] = hit
        return hit[1]

    def _decode(self, xb_y, cache: RNNCache):
        """One cached token: xb_y [B,1,2R] (hawk/hawk.py:168-179,193-199)."""
        conv = self.conv1d
        gi, ga_ = self.rg_lru_input_gate, self.rg_lru_a_gate
        state = cache.recc_state[:, 0]
        cw, cb, lam = self._fp32("w", conv.w), self._fp32("b", conv.b), self._fp32("lam", self.rg_lru_a_param)
        if gi.block_width <= 128 and conv.temporal_width <= 4:
            # conv step, both gate projections, RG-LRU step and gelu(y) * h in one launch
            out = ops.decode_block_step(xb_y[:, 0], cache.conv_state, cw, cb, gi.w, ga_.w, self._fp32("bx", gi.b),
                                        self._fp32("ba", ga_.b), lam, state)
            cache.current_cache_size = 1
            return self.resid_proj(out[:, None])
        xb, y = xb_y.chunk(2, dim=-1)
        xc = ops.decode_conv_step(xb[:, 0], cache.conv_state, cw, cb)
        gx, ga = ops.block_diag_gates(xc, gi.w, gi.b, ga_.w, ga_.b)
        h = ops.decode_rglru_step(xc, gx, ga, lam, state)
        cache.current_cache_size = 1
        return self.resid_proj(ops.gelu_mul(y, h[:, None]))

    def forward(self, x, layer_past: Optional[RNNCache] = None):
        cached = layer_past is not None and self.use_cache and layer_past.current_cache_size > 0
        xb_y = self.input_xy(x)
        xb, y = xb_y.chunk(2, dim=-1)
        if cached:
            assert x.shape[1] == 1, "cached decode takes one token per call"
            return self._decode(xb_y, layer_past), layer_past

        # conv -> gates -> scan -> gelu(y) * h as one autograd node; the gate biases go to the scan kernel,
        # which adds them for free and sums their gradients
        conv = self.conv1d
        gate_bias = torch.stack((self.rg_lru_input_gate.b.reshape(-1), self.rg_lru_a_gate.b.reshape(-1))).float()
        out, h = ops.recurrent_core(xb_y, self._fp32("w", conv.w) if not conv.w.requires_grad else conv.w.float(),
                                    self._fp32("b", conv.b) if not conv.b.requires_grad else conv.b.float(),
                                    self.rg_lru_input_gate.w, self.rg_lru_a_gate.w, gate_bias,
                                    self.rg_lru_a_param.float())
        cache = None
        if self.use_cache:
            assert layer_past is not None, "use_cache=True needs an RNNCache per layer"
            keep = layer_past.conv_cache_size
            tail = xb[:, -keep:]
            if tail.shape[1] < keep:  # prompt shorter than the conv history: zero history before it
                tail = F.pad(tail, (0, 0, keep - tail.shape[1], 0))
            layer_past.conv_state.copy_(tail)
            layer_past.update_cache(h[:, -1:])
            cache = layer_past
        return self.resid_proj(out), cache


class RNNLayer(nn.Module):
    """Pre-norm residual pair: recurrent block, then MLP (hawk/hawk.py:206-236)."""

    def __init__(self, config: HawkConfig, use_cache: bool = False):
        super().__init__()
        self.recc = Hawk(config, use_cache)
        self.mlp = MLP(config)
        self.input_norm = RMSNorm(config.hidden_size)
        self.post_recurrent_norm = RMSNorm(config.hidden_size)

    def step(self, residual, pending, layer_past: Optional[RNNCache] = None):
        """The layer on a residual stream whose last branch output `pending` has not been added yet
        (None for the first layer).  Returns (residual, pending, cache) in the same form."""
        residual, normed = self.input_norm.add_forward(residual, pending)
        mixed, cache = self.recc(normed, layer_past)
        residual, normed = self.post_recurrent_norm.add_forward(residual, mixed)
        return residual, self.mlp(normed), cache

    def forward(self, hidden_states, layer_past: Optional[RNNCache] = None):
        residual, pending, cache = self.step(hidden_states, None, layer_past)
        return residual + pending, cache


class HawkModel(nn.Module):
    """hawk/hawk.py:239-303."""

    def __init__(self, config: HawkConfig, use_cache: bool = False):
        super().__init__()
        self.config = config
        self.use_cache = use_cache
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList(RNNLayer(config, use_cache) for _ in range(config.num_hidden_layers))
        self.norm = RMSNorm(config.hidden_size)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        _lecun_normal_(self.embed_tokens.weight, config.hidden_size)
        nn.init.zeros_(self.lm_head.weight)

    def new_caches(self, batch_size: int, device=None, dtype: torch.dtype = torch.bfloat16) -> List[RNNCache]:
        device = device or self.embed_tokens.weight.device
        return [RNNCache(self.config.recurrent_size, device, self.config.conv_width, batch_size, dtype)
                for _ in self.layers]

    def forward(self, input_ids, labels=None, layer_past: Optional[List[Optional[RNNCache]]] = None):
        if layer_past is None:
            layer_past = [None] * len(self.layers)
        hidden = self.embed_tokens(input_ids)
        pending = None  # branch output not yet added to the residual stream: folded into the next norm
        caches = []
        for layer, past in zip(self.layers, layer_past):
            hidden, pending, cache = layer.step(hidden, pending, past)
            caches.append(cache)
        _, hidden = self.norm.add_forward(hidden, pending)
        if self.use_cache:
            return self.lm_head(hidden), caches
        if labels is None:
            return self.lm_head(hidden)
        # next-token loss: position t predicts token t+1 (hawk/hawk.py:291-300)
        act = hidden[..., :-1, :].reshape(-1, hidden.shape[-1])
        targets = labels[..., 1:].reshape(-1)
        return ops.fused_cross_entropy(self.lm_head.weight, act, targets)


# the configurations named by the benchmark contract
def readme_config() -> HawkConfig:
    """The reference README's model (its `post_norm` argument does not exist in HawkConfig)."""
    return HawkConfig(vocab_size=32000, hidden_size=512, intermediate_size=1024, num_hidden_layers=8,
                      recurrent_size=512, num_blocks=16, conv_width=4)


def hawk_1b_config() -> HawkConfig:
    """~1.35 B parameters: hidden = recurrent = 2048, intermediate 6144, 24 layers."""
    return HawkConfig(vocab_size=32000, hidden_size=2048, intermediate_size=6144, num_hidden_layers=24,
                      recurrent_size=2048, num_blocks=16, conv_width=4)
