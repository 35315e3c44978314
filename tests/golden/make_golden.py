"""Generates the golden fixtures in this folder by running the UNMODIFIED reference.

Run once where the reference checkout is available (it is not needed, and not
read, by any test):

    TRITON_INTERPRET=1 TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py /path/to/hawk-pytorch

What is produced (all float32 / int64 arrays in .npz, a few hundred KB total):

  scan_triton_interp.npz  the reference Triton kernels (hawk/scan_fused.py) executed by
                          the Triton CPU interpreter on fp32 inputs: h, dx, dgx, dga, dlam.
                          The interpreter rounds the kernels' bf16 stores by truncation.
  conv1d_ref.npz          hawk/external.py Conv1D forward + autograd backward on a strided view.
  linear_ce_ref.npz       hawk/fused_cross_entropy.py CrossEntropyLoopedFused (eager) loss, dW, dact,
                          N > 2048 so the chunk loop runs twice.
  model_ref.npz           hawk/hawk.py HawkModel (tiny config, fp32, CPU).  Its Triton scan cannot run
                          without a GPU, so hawk.hawk.fused_linear_scan is rebound to the fp32
                          restatement in oracle/scan.py wrapped in an autograd.Function; every other
                          line of the model is the reference's.  Holds the state dict, the loss at
                          the reference init (= ln V), and loss + gradients after de-zeroing.
  decode_ref.npz          HawkModel(use_cache=True): prefill of 5 tokens then 3 cached single-token
                          steps (batch 1, the only batch the reference cache accepts), logits per call.
"""
from __future__ import annotations

import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py <path to a checkout of fattorib/hawk-pytorch>")
ref_path = sys.argv[1]
sys.path.insert(0, ref_path)

import hawk  # noqa: E402  (the reference package)
import hawk.hawk as ref_hawk  # noqa: E402
from hawk.cache import RNNCache  # noqa: E402
from hawk.external import Conv1D, rnn_param_init  # noqa: E402
from hawk.fused_cross_entropy import CrossEntropyLoopedFused  # noqa: E402
from hawk.scan_fused import sequential_scan_backward, sequential_scan_forward  # noqa: E402

from oracle import model as omodel  # noqa: E402
from oracle import scan as oscan  # noqa: E402


def np_(t):
    return t.detach().cpu().numpy()


def make_scan():
    out = {}
    for tag, (B, T, D, scale) in {"a": (2, 12, 128, 1.0), "b": (1, 5, 64, 4.0), "c": (3, 2, 64, 1.0)}.items():
        g = torch.Generator().manual_seed(100 + ord(tag))
        x, gx, ga, go = (torch.randn(B, T, D, generator=g) * scale for _ in range(4))
        lam = rnn_param_init(torch.empty(D), 0.9, 0.999)
        h = sequential_scan_forward(x, gx, ga, lam)
        dx, dgx, dga, dlam = sequential_scan_backward(x, gx, ga, lam, h, go)
        for k, v in dict(x=x, gx=gx, ga=ga, go=go, lam=lam, h=h, dx=dx, dgx=dgx, dga=dga, dlam=dlam).items():
            out[f"{tag}_{k}"] = np_(v)
    np.savez_compressed(os.path.join(HERE, "scan_triton_interp.npz"), **out)


def make_conv():
    torch.manual_seed(7)
    B, T, D = 2, 9, 24
    conv = Conv1D(width=D, temporal_width=4)
    with torch.no_grad():
        conv.b.normal_()
        conv.w.normal_()
    xy = torch.randn(B, T, 2 * D, requires_grad=True)
    x = xy[..., :D]  # strided view, as torch.chunk gives in hawk.py:166
    y = conv(x)
    go = torch.randn_like(y)
    y.backward(go)
    out = dict(x=np_(x), w=np_(conv.w), b=np_(conv.b), y=np_(y), go=np_(go),
               dx=np_(xy.grad[..., :D]), dw=np_(conv.w.grad), db=np_(conv.b.grad))
    # T shorter than the temporal width
    xs = torch.randn(1, 2, D)
    out["short_x"] = np_(xs)
    out["short_y"] = np_(conv(xs))
    np.savez_compressed(os.path.join(HERE, "conv1d_ref.npz"), **out)


def make_ce():
    torch.manual_seed(11)
    N, H, V = 2100, 32, 97
    w = (torch.randn(V, H) / H**0.5).requires_grad_(True)
    act = torch.randn(N, H, requires_grad=True)
    labels = torch.randint(0, V, (N,))
    labels[0] = 0
    labels[1] = V - 1
    loss = CrossEntropyLoopedFused.apply(w, act, labels)
    (2.5 * loss).backward()
    np.savez_compressed(os.path.join(HERE, "linear_ce_ref.npz"), w=np_(w), act=np_(act), labels=np_(labels),
                        loss=np_(loss), dw=np_(w.grad), dact=np_(act.grad), upstream=np.float32(2.5))


class _OracleScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gx, ga, lam):
        h = oscan.rglru_scan_fwd(x, gx, ga, lam)
        ctx.save_for_backward(x, gx, ga, lam, h)
        return h

    @staticmethod
    def backward(ctx, go):
        x, gx, ga, lam, h = ctx.saved_tensors
        return oscan.rglru_scan_bwd(x, gx, ga, lam, h, go.contiguous())


def make_model():
    ref_hawk.fused_linear_scan = _OracleScan.apply
    ref_hawk.fused_cross_entropy = lambda w, a, l: CrossEntropyLoopedFused.apply(w, a, l)
    cfg = hawk.HawkConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                          recurrent_size=64, num_blocks=4, conv_width=4)
    torch.manual_seed(0)
    model = hawk.HawkModel(cfg)
    ids = torch.randint(1, cfg.vocab_size, (2, 17))
    out = {"ids": np_(ids), "cfg": np.array([96, 64, 128, 2, 64, 4, 4])}
    loss0 = model(ids, ids)
    loss0.backward()
    out["loss_init"] = np_(loss0)
    out["lm_head_grad_init"] = np_(model.lm_head.weight.grad)
    sd = {k: v.detach().clone() for k, v in model.state_dict().items()}
    sd = omodel.dezero(sd, seed=1)
    # non-zero conv / gate biases so that every parameter matters
    g = torch.Generator().manual_seed(2)
    for k in sorted(sd):
        if k.endswith("conv1d.b") or k.endswith("_gate.b"):
            sd[k] = 0.1 * torch.randn(sd[k].shape, generator=g)
    model.load_state_dict(sd)
    model.zero_grad()
    loss1 = model(ids, ids)
    loss1.backward()
    out["loss_dezero"] = np_(loss1)
    for k, v in sd.items():
        out["sd/" + k] = np_(v)
    for k, p in model.named_parameters():
        out["grad/" + k] = np_(p.grad)
    out["logits_dezero"] = np_(model(ids))
    np.savez_compressed(os.path.join(HERE, "model_ref.npz"), **out)
    return cfg, sd


def make_decode(cfg, sd):
    model = hawk.HawkModel(cfg, use_cache=True)
    model.load_state_dict(sd)
    torch.manual_seed(5)
    ids = torch.randint(1, cfg.vocab_size, (1, 8))
    caches = [RNNCache(cfg.recurrent_size, torch.device("cpu"), cfg.conv_width) for _ in range(cfg.num_hidden_layers)]
    out = {"ids": np_(ids)}
    with torch.no_grad():
        logits, caches = model(ids[:, :5], layer_past=caches)
        out["prefill_logits"] = np_(logits)
        for s in range(3):
            logits, caches = model(ids[:, 5 + s : 6 + s], layer_past=caches)
            out[f"step{s}_logits"] = np_(logits)
        out["final_recc_state0"] = np_(caches[0].recc_state.float())
        out["final_conv_state0"] = np_(caches[0].conv_state.float())
    np.savez_compressed(os.path.join(HERE, "decode_ref.npz"), **out)


if __name__ == "__main__":
    make_scan()
    make_conv()
    make_ce()
    cfg, sd = make_model()
    make_decode(cfg, sd)
    print("golden fixtures written to", HERE)
