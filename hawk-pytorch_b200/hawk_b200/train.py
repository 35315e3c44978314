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


class FusedAdamW(torch.optim.Optimizer):
    """torch.optim.AdamW's update (decoupled weight decay, bias correction) with one kernel per fp32
    parameter tensor that also writes the bf16 copy of the updated weight for the model's `Linear`
    layers (`shadow_modules`: modules with `.weight`, `.weight_bf16`, `.weight_bf16_version`), so the next
    forward casts nothing.  State keys follow torch.optim.AdamW (`step`, `exp_avg`, `exp_avg_sq`)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, shadow_modules=()):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._shadow = {id(m.weight): m for m in shadow_modules}

    @torch.no_grad()
    def step(self, closure=None):
        from . import _lib, ops
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        lib = _lib.load()
        touched = []
        for group in self.param_groups:
            b1, b2 = group["betas"]
            lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                g = p.grad
                if g is None:
                    continue
                st = self.state[p]
                if not st:
                    self._init_state(p, st)
                st["step"] += 1
                if not g.is_contiguous():
                    g = g.contiguous()
                # pointers of p, m, v and the bf16 copy are fixed for the life of the state: one ctypes
                # call per tensor with cached addresses keeps the host side of 300+ launches to ~2 ms
                p_ptr, m_ptr, v_ptr, wb_ptr, n, dev = st["_args"]
                if p_ptr != p.data_ptr():  # the parameter was moved or re-allocated since the state was made
                    self._bind(p, st)
                    p_ptr, m_ptr, v_ptr, wb_ptr, n, dev = st["_args"]
                if dev != torch.cuda.current_device():
                    with torch.cuda.device(dev):
                        rc = lib.hawk_adamw_step(p_ptr, g.data_ptr(), m_ptr, v_ptr, wb_ptr, n, lr, b1, b2, eps, wd,
                                                 st["step"], torch.cuda.current_stream().cuda_stream)
                else:
                    rc = lib.hawk_adamw_step(p_ptr, g.data_ptr(), m_ptr, v_ptr, wb_ptr, n, lr, b1, b2, eps, wd,
                                             st["step"], torch.cuda.current_stream().cuda_stream)
                _lib.check(rc, "hawk_adamw_step")
                touched.append(p)
        if touched:
            torch.autograd.graph.increment_version(touched)  # the kernels wrote p behind autograd's back
            for p in touched:
                mod = self._shadow.get(id(p))
                if mod is not None:
                    mod.weight_bf16, mod.weight_bf16_version = self.state[p]["_shadow"], p._version
            if ops.LOG.enabled:
                ops.LOG.counts["adamw_step"] = ops.LOG.counts.get("adamw_step", 0) + len(touched)
        return loss

    def _init_state(self, p, st):
        assert p.is_cuda and p.dtype == torch.float32 and p.is_contiguous(), "FusedAdamW: contiguous fp32 CUDA parameters"
        st["step"] = 0
        st["exp_avg"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
        st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
        self._bind(p, st)

    def _bind(self, p, st):
        """(Re)build what is derived from the state: the bf16 copy's buffer and the cached addresses."""
        for k in ("exp_avg", "exp_avg_sq"):
            if st[k].device != p.device or not st[k].is_contiguous():
                st[k] = st[k].to(p.device).contiguous()
        wb = None
        if id(p) in self._shadow:
            wb = torch.empty(p.shape, dtype=torch.bfloat16, device=p.device)
        st["_shadow"] = wb
        st["_args"] = (p.data_ptr(), st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr(),
                       None if wb is None else wb.data_ptr(), p.numel(), p.device.index)

    def state_dict(self):
        sd = super().state_dict()  # cached addresses and the bf16 copies are derived, not state
        sd["state"] = {k: {kk: vv for kk, vv in v.items() if not kk.startswith("_")} for k, v in sd["state"].items()}
        return sd

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        for p, st in self.state.items():
            if st:
                st["step"] = int(st["step"])
                self._bind(p, st)


class CommTimeline:
    """Times the gradient all-reduce of every DDP bucket against the backward pass (CUDA events): when the
    bucket became ready on the compute stream, when its all-reduce finished on the communication stream.
    `summary()` after a step gives how long the all-reduces were in flight and how far the last one ran past
    the moment the last bucket became ready, i.e. past the end of the backward computation (the part of the
    communication the step could not hide; DDP makes the compute stream wait for it before the optimiser)."""

    def __init__(self):
        self.ready = []        # ready events in the order the buckets were handed over
        self.records = []      # (bucket index, bytes, ready event, done event)

    def reset(self):
        self.ready, self.records = [], []

    def summary(self):
        torch.cuda.synchronize()
        if not self.records:
            return None
        first, last = self.ready[0], self.ready[-1]
        spans = [r[2].elapsed_time(r[3]) for r in self.records]
        return {"buckets": len(self.records), "bytes": sum(r[1] for r in self.records),
                "ready_to_done_ms": {"max": max(spans), "sum": sum(spans)},
                "first_to_last_bucket_ready_ms": first.elapsed_time(last),
                "exposed_tail_ms": max(0.0, max(last.elapsed_time(r[3]) for r in self.records))}


def _comm_hook(timeline: Optional[CommTimeline], compress_bf16: bool):
    """DDP communication hook: the default all-reduce (averaging), optionally in bf16, optionally timed."""
    from torch.distributed.algorithms.ddp_comm_hooks import default_hooks

    def hook(state, bucket):
        if timeline is not None:
            ready = torch.cuda.Event(enable_timing=True)
            ready.record()
            timeline.ready.append(ready)
            nbytes = bucket.buffer().numel() * bucket.buffer().element_size()
            index = bucket.index()
        fut = (default_hooks.bf16_compress_hook if compress_bf16 else default_hooks.allreduce_hook)(state, bucket)
        if timeline is None:
            return fut

        def done(f):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()  # runs with the communication stream current, after the bucket's all-reduce
            timeline.records.append((index, nbytes, ready, ev))
            return f.value()[0]
        return fut.then(done)
    return hook


class Trainer:
    """Model + AdamW (+ DDP when world_size > 1).  `step(ids)` runs forward (bf16 autocast, fused
    cross-entropy with labels = inputs), backward, gradient all-reduce and the optimiser update.
    `grad_comm_dtype`: torch.float32 (default: the gradients are all-reduced as they are) or torch.bfloat16
    (each bucket is rounded to bf16 for the all-reduce and restored: half the NVLink bytes).
    `timeline`: a CommTimeline that the step fills (multi-GPU only).  `check_status_every`: see below."""

    def __init__(self, config: HawkConfig, device, seed: int = 0, lr: float = 3e-4, world_size: int = 1,
                 autocast: bool = True, bucket_cap_mb: int = 256, grad_comm_dtype: torch.dtype = torch.float32,
                 timeline: Optional[CommTimeline] = None, check_status_every: int = 100):
        torch.manual_seed(seed)  # same seed on every rank: identical replicas
        self.device = torch.device(device)
        self.model = HawkModel(config).to(self.device)
        self.autocast = autocast and self.device.type == "cuda"
        self.ddp = None
        self.steps_done = 0
        # every this many steps the device status word of the tensor-core kernels is read back (one host sync):
        # a kernel that gave up a bounded wait then raises here instead of training on (its loss is NaN anyway)
        self.check_status_every = check_status_every
        self.timeline = timeline if world_size > 1 else None
        if world_size > 1:
            from torch.nn.parallel import DistributedDataParallel as DDP
            ids = [self.device.index] if self.device.type == "cuda" else None
            self.ddp = DDP(self.model, device_ids=ids, gradient_as_bucket_view=True, bucket_cap_mb=bucket_cap_mb)
            assert grad_comm_dtype in (torch.float32, torch.bfloat16)
            if self.device.type == "cuda" and (self.timeline is not None or grad_comm_dtype == torch.bfloat16):
                self.ddp.register_comm_hook(None, _comm_hook(self.timeline, grad_comm_dtype == torch.bfloat16))
        if self.device.type == "cuda":
            from .model import Linear
            shadows = [m for m in self.model.modules() if isinstance(m, Linear) and m.bias is None] if self.autocast else []
            self.opt = FusedAdamW(self.model.parameters(), lr=lr, weight_decay=0.1, shadow_modules=shadows)
        else:
            self.opt = torch.optim.AdamW(self.model.parameters(), lr=lr, weight_decay=0.1,
                                         fused=self.device.type == "cuda")

    def step(self, ids: torch.Tensor, after_backward=None, sync_gradients: bool = True) -> torch.Tensor:
        """One training step; `after_backward(loss)`, when given, runs between the backward pass (gradients
        all-reduced) and the optimiser update, e.g. to inspect gradients.  `sync_gradients=False` (multi-GPU
        measurement only: the replicas diverge) skips the gradient all-reduce, so that a rank's own compute
        time can be told apart from communication and from waiting for slower ranks."""
        net = self.ddp if self.ddp is not None else self.model
        if not sync_gradients and self.ddp is not None:
            with self.ddp.no_sync():
                with torch.autocast(self.device.type, dtype=torch.bfloat16, enabled=self.autocast):
                    loss = net(ids, ids)
                loss.backward()
            self.opt.step()
            self.opt.zero_grad(set_to_none=True)
            self.steps_done += 1
            return loss.detach()
        with torch.autocast(self.device.type, dtype=torch.bfloat16, enabled=self.autocast):
            loss = net(ids, ids)
        if self.timeline is not None:
            self.timeline.reset()
        loss.backward()
        if after_backward is not None:
            after_backward(loss.detach())
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        self.steps_done += 1
        if self.check_status_every > 0 and self.steps_done % self.check_status_every == 0 and self.device.type == "cuda":
            from . import ops
            ops.check_device_status(self.device)
        return loss.detach()
