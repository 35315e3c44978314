"""Worker of tests/test_dp_gloo.py: one data-parallel rank on CPU over gloo.  The product has no CPU
kernels, so this TEST substitutes oracle statements for the three operators before training."""
import os
import sys

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "hawk-pytorch_b200"))

import hawk_b200.model as M  # noqa: E402
from hawk_b200 import train  # noqa: E402
from oracle import model as omodel  # noqa: E402


def _scan_with_bias(x, gx, ga, lam, h0=None, gate_bias=None):
    """The scan's gate_bias is the broadcast bias add of the gate projections moved inside it."""
    if gate_bias is not None:
        gx, ga = gx + gate_bias[0], ga + gate_bias[1]
    return omodel.scan(x, gx, ga, lam)


def _recurrent_core(xy, conv_w, conv_b, wx, wa, gate_bias, lam):
    """hawk/hawk.py:164-166,181-199 from oracle statements: (gelu(y) * h, h)."""
    xb, y = xy.chunk(2, dim=-1)
    xc = omodel.conv1d(xb, conv_w, conv_b)
    nb, bw, _ = wx.shape
    gx = omodel.block_diag_linear(xc, wx, gate_bias[0].view(nb, bw))
    ga = omodel.block_diag_linear(xc, wa, gate_bias[1].view(nb, bw))
    h = omodel.scan(xc, gx, ga, lam)
    return F.gelu(y) * h, h


# oracle statements standing in for the kernels (the product has no CPU path; only tests do this)
SUBSTITUTES = {
    "fused_linear_scan": _scan_with_bias,
    "recurrent_core": _recurrent_core,
    "fused_cross_entropy": lambda w, a, l: F.cross_entropy(F.linear(a, w), l),
    "rms_norm": lambda x, w, eps=1e-6, out_dtype=None: omodel.rms_norm(x, w),
    "add_rms_norm": lambda r, d, w, eps=1e-6, out_dtype=None: (
        (r, omodel.rms_norm(r, w)) if d is None else (r + d, omodel.rms_norm(r + d, w))),
    "geglu": lambda gu: F.gelu(gu.chunk(2, -1)[0]) * gu.chunk(2, -1)[1],
    "gelu_mul": lambda a, b: F.gelu(a) * b,
    "block_diag_gates": lambda x, wx, bx, wa, ba: (omodel.block_diag_linear(x, wx, 0.0 if bx is None else bx),
                                                   omodel.block_diag_linear(x, wa, 0.0 if ba is None else ba)),
}
CONV_FORWARD = lambda self, x: omodel.conv1d(x, self.w, self.b)  # noqa: E731


def patch_ops(setattr_=setattr):
    """In a worker process: plain setattr.  Inside pytest: pass monkeypatch.setattr so it is undone."""
    for name, fn in SUBSTITUTES.items():
        setattr_(M.ops, name, fn)
    setattr_(M.ops.Conv1D, "forward", CONV_FORWARD)


def make_trainer(world):
    cfg = M.HawkConfig(64, 32, 64, 2, 32, 4, 4)
    tr = train.Trainer(cfg, "cpu", seed=0, lr=1e-2, world_size=world, autocast=False)
    sd = omodel.dezero(dict(tr.model.state_dict()), seed=1)  # so that every parameter gets a gradient
    tr.model.load_state_dict(sd)
    return tr


def data(step):
    g = torch.Generator().manual_seed(100 + step)
    return torch.randint(1, 64, (4, 12), generator=g)  # the GLOBAL batch of this step


if __name__ == "__main__":
    out_path = sys.argv[1]
    fail_rank = int(sys.argv[2]) if len(sys.argv) > 2 else -1
    unsynced_tail = len(sys.argv) > 3 and sys.argv[3] == "unsynced"  # one more step without the all-reduce
    patch_ops()
    rank, _, world = train.init_distributed("gloo")
    tr = make_trainer(world)
    losses = []
    for step in range(3):
        if rank == fail_rank and step == 1:
            os._exit(17)  # a rank that dies between steps: the others must fail, not hang
        ids = data(step).chunk(world, dim=0)[rank]  # batch sharding: rank r takes its slice
        losses.append(float(tr.step(ids)))
    synced = {k: v.detach().clone() for k, v in tr.model.state_dict().items()}
    if unsynced_tail:
        tr.step(data(3).chunk(world, dim=0)[rank], sync_gradients=False)
        torch.save({"synced": synced, "after": {k: v.detach().clone() for k, v in tr.model.state_dict().items()}},
                   f"{out_path}.tail.{rank}")
    torch.save({"losses": losses, "params": {k: v.detach().clone() for k, v in tr.model.state_dict().items()}},
               f"{out_path}.{rank}")
