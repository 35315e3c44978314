"""Worker of tests/test_gpu_dp_nccl.py: one data-parallel rank on its own GPU (NCCL), real kernels.
Writes the per-step losses, the gradients of the first step (after the all-reduce) and the final parameters."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "hawk-pytorch_b200"))

import hawk_b200.model as M  # noqa: E402
from hawk_b200 import ops, train  # noqa: E402
from oracle import model as omodel  # noqa: E402

CFG = (1024, 128, 256, 2, 128, 16, 4)
GLOBAL_BATCH, SEQ = 8, 96


def data(step):
    g = torch.Generator().manual_seed(500 + step)
    return torch.randint(1, CFG[0], (GLOBAL_BATCH, SEQ), generator=g)  # the GLOBAL batch of this step


def make_trainer(device, world, timeline=None):
    tr = train.Trainer(M.HawkConfig(*CFG), device, seed=0, lr=1e-3, world_size=world, timeline=timeline)
    sd = omodel.dezero({k: v.cpu() for k, v in tr.model.state_dict().items()}, seed=1)  # every parameter gets a gradient
    tr.model.load_state_dict(sd)
    return tr


def run(tr, rank, world, steps=3):
    losses, grads = [], {}

    def grab(_loss):
        if not grads:
            grads.update({k: p.grad.detach().float().cpu().clone() for k, p in tr.model.named_parameters()})
    for step in range(steps):
        ids = data(step).chunk(world, dim=0)[rank].to(tr.device)
        losses.append(float(tr.step(ids, after_backward=grab)))
    ops.check_device_status()
    return {"losses": losses, "grads": grads,
            "params": {k: v.detach().float().cpu().clone() for k, v in tr.model.state_dict().items()}}


if __name__ == "__main__":
    out_path = sys.argv[1]
    rank, local_rank, world = train.init_distributed("nccl")
    torch.cuda.set_device(local_rank)
    tl = train.CommTimeline()
    tr = make_trainer(torch.device("cuda", local_rank), world, timeline=tl)
    res = run(tr, rank, world)
    res["comm"] = tl.summary()
    torch.save(res, f"{out_path}.{rank}")
    torch.distributed.destroy_process_group()
