"""Batch data-parallel training harness: one process per GPU, parameters replicated, the global
batch split across ranks, NCCL used only for the gradient all-reduce (bucketed and overlapped with
the backward pass by DistributedDataParallel).  The reference has no distributed code; this is the
harness the multi-GPU benchmark and tests drive."""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .model import HawkConfig, HawkModel


def dist_env():
    """(rank, local_rank, world_size) from the torchrun environment; (0, 0, 1) when launched plainly."""
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)))


def init_distributed(backend: Optional[str] = None) -> tuple:
    rank, local_rank, world = dist_env()
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, local_rank, world


class Trainer:
    """Model + AdamW (+ DDP when world_size > 1).  `step(ids)` runs forward (bf16 autocast, fused
    cross-entropy with labels = inputs), backward, gradient all-reduce and the optimiser update."""

    def __init__(self, config: HawkConfig, device, seed: int = 0, lr: float = 3e-4, world_size: int = 1,
                 autocast: bool = True, bucket_cap_mb: int = 256):
        torch.manual_seed(seed)  # same seed on every rank: identical replicas
        self.device = torch.device(device)
        self.model = HawkModel(config).to(self.device)
        self.autocast = autocast and self.device.type == "cuda"
        self.ddp = None
        if world_size > 1:
            from torch.nn.parallel import DistributedDataParallel as DDP
            ids = [self.device.index] if self.device.type == "cuda" else None
            self.ddp = DDP(self.model, device_ids=ids, gradient_as_bucket_view=True, bucket_cap_mb=bucket_cap_mb)
        fused = self.device.type == "cuda"
        self.opt = torch.optim.AdamW(self.model.parameters(), lr=lr, weight_decay=0.1, fused=fused)

    def step(self, ids: torch.Tensor) -> torch.Tensor:
        net = self.ddp if self.ddp is not None else self.model
        with torch.autocast(self.device.type, dtype=torch.bfloat16, enabled=self.autocast):
            loss = net(ids, ids)
        loss.backward()
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        return loss.detach()
