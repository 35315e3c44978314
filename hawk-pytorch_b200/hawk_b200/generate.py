"""Cached decoding for any batch size, with the per-token step replayed as one CUDA graph.

The reference decodes one sequence at a time through ~15 eager launches per layer per token
(hawk/hawk.py:168-199, hawk/cache.py); a single decode step of a 24-layer model is launch bound.
Here the whole step (embedding, 24 x [norm, projection, fused conv step, gate GEMMs, fused RG-LRU
step, gelu*h, projections, MLP], final norm, lm_head) is captured once for a fixed batch size and
replayed per token: the recurrent and conv caches are updated in place by the kernels, the token
ids and logits live in static buffers.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .model import HawkModel, RNNCache


class GraphedDecoder:
    """`prefill(ids)` runs the prompt eagerly and fills the caches; `step(token_ids)` replays the
    captured single-token step and returns logits [B, 1, V] (a static buffer, overwritten per call)."""

    def __init__(self, model: HawkModel, batch_size: int, cache_dtype: torch.dtype = torch.bfloat16,
                 autocast: bool = True, use_graph: bool = True):
        assert model.use_cache, "construct the model with use_cache=True"
        self.model = model.eval()
        self.batch_size = batch_size
        self.autocast = autocast
        self.use_graph = use_graph
        self.device = model.embed_tokens.weight.device
        self.caches: List[RNNCache] = model.new_caches(batch_size, dtype=cache_dtype)
        self._ids = torch.zeros(batch_size, 1, dtype=torch.int64, device=self.device)
        self._logits: Optional[torch.Tensor] = None
        self._graph: Optional[torch.cuda.CUDAGraph] = None

    def _forward(self, ids):
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16, enabled=self.autocast):
            logits, _ = self.model(ids, layer_past=self.caches)
        return logits

    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        assert ids.shape[0] == self.batch_size
        for c in self.caches:
            c.current_cache_size = 0
        return self._forward(ids)

    def _capture(self):
        # warm up on a side stream (library handles, autotuning, allocator pools), keeping the cache
        # contents: the warm-up steps must not advance the state
        saved = [(c.recc_state.clone(), c.conv_state.clone()) for c in self.caches]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._forward(self._ids)
        torch.cuda.current_stream().wait_stream(side)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._logits = self._forward(self._ids)
        for c, (r, k) in zip(self.caches, saved):
            c.recc_state.copy_(r)
            c.conv_state.copy_(k)

    def step(self, token_ids: torch.Tensor) -> torch.Tensor:
        assert all(c.current_cache_size > 0 for c in self.caches), "call prefill() first"
        if not self.use_graph:
            return self._forward(token_ids)
        if self._graph is None:
            self._capture()
        self._ids.copy_(token_ids)
        self._graph.replay()
        return self._logits
