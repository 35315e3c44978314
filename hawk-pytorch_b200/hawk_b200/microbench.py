"""Times one operator of this library in isolation (CUDA events, median of N launches).

    python -m hawk_b200.microbench scan      [--B 8 --T 4096 --D 2048 --dtype bf16]
    python -m hawk_b200.microbench scan_gelu [--B 8 --T 4096 --D 2048 --dtype bf16]   # scan with gelu(y)*h fused in
    python -m hawk_b200.microbench gates     [--B 8 --T 4096 --D 2048 --bw 128]       # both gate projections
    python -m hawk_b200.microbench conv1d    [--B 8 --T 4096 --D 2048 --dtype bf16]
    python -m hawk_b200.microbench linear_ce [--N 32760 --H 2048 --V 32000]
    python -m hawk_b200.microbench glue      [--N 32768 --H 2048 --J 6144]   # gelu(a)*b and add+RMSNorm, both ways
    python -m hawk_b200.microbench decode    [--B 256 --D 2048 --layers 24]
    python -m hawk_b200.microbench decode_model [--B 256]   # one cached token of the 1.35 B model, eager vs CUDA graph

Prints one JSON line per kernel with the achieved rate against its algorithmic work:
scan 8 (forward) / 16 (backward) bytes per element in bf16 (12 / 20 with the fused gelu(y)*h epilogue), gate
projections 6 / 14, conv1d 4 / 6, linear_ce 6*N*H*V flop,
decode 8*B*D*elem bytes per step; glue: the tensors each kernel must read and write once (gelu(a)*b:
3 / 5 bf16 tensors of N x J; add+RMSNorm with an fp32 residual stream and bf16 branch: 12 / 16 bytes per
element).  Inputs are seeded normal draws; Lambda sits on the reference's
0.9..0.999 ring.  Working sets beyond the 126 MB L2 need no flush between launches; smaller ones
are bracketed by a flush write (`--flush`).
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from . import ops
from .model import ring_init_


def _time(fn, iters, warmup, flush=None):
    """Median device time of one launch.  Launches are queued back to back and bracketed pairwise by
    events, so the stream never runs dry (an idle stream would add host launch latency to the interval)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in evs)
    return ts[len(ts) // 2]


def _emit(name, ms, work, unit, **extra):
    rate = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
    print(json.dumps({"kernel": name, "ms": round(ms, 5), "rate": round(rate, 1), "unit": unit, **extra}), flush=True)
    return rate


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["scan", "scan_gelu", "gates", "conv1d", "linear_ce", "glue", "decode", "decode_model"])
    ap.add_argument("--bw", type=int, default=128)
    ap.add_argument("--J", type=int, default=6144)
    ap.add_argument("--B", type=int, default=None)
    ap.add_argument("--T", type=int, default=4096)
    ap.add_argument("--D", type=int, default=2048)
    ap.add_argument("--N", type=int, default=8 * 4095)
    ap.add_argument("--H", type=int, default=2048)
    ap.add_argument("--V", type=int, default=32000)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--flush", action="store_true")
    a = ap.parse_args(argv)
    if a.B is None:
        a.B = 256 if a.op.startswith("decode") else 8
    dev = torch.device("cuda")
    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    es = 2 if a.dtype == "bf16" else 4
    g = torch.Generator(device="cuda").manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if a.flush else None
    shape = {"B": a.B, "T": a.T, "D": a.D, "dtype": a.dtype}

    if a.op == "scan":
        x, gx, ga, go = (torch.randn(a.B, a.T, a.D, generator=g, device=dev).to(dt) for _ in range(4))
        lam = ring_init_(torch.empty(a.D)).to(dev)
        n = a.B * a.T * a.D
        gb = 0.1 * torch.randn(2, a.D, generator=g, device=dev)  # gate biases, as the model passes them
        h = ops.scan_fwd(x, gx, ga, lam, None, gb)
        tf = _time(lambda: ops.scan_fwd(x, gx, ga, lam, None, gb), a.iters, a.warmup, flush)
        tb = _time(lambda: ops.scan_bwd(x, gx, ga, lam, None, gb, h, go), a.iters, a.warmup, flush)
        _emit("scan_fwd", tf, 4 * es * n, "GB/s", **shape)
        _emit("scan_bwd", tb, 8 * es * n, "GB/s", **shape)
        _emit("scan_fwd+bwd", tf + tb, 12 * es * n, "GB/s", **shape)
    elif a.op == "scan_gelu":
        x, gx, ga, go = (torch.randn(a.B, a.T, a.D, generator=g, device=dev).to(dt) for _ in range(4))
        xy = torch.randn(a.B, a.T, 2 * a.D, generator=g, device=dev).to(dt)
        y = xy[..., a.D:]  # the strided half the model passes
        dxy = torch.empty_like(xy)
        lam = ring_init_(torch.empty(a.D)).to(dev)
        n = a.B * a.T * a.D
        gb = 0.1 * torch.randn(2, a.D, generator=g, device=dev)
        h, _ = ops.scan_gelu_fwd(x, gx, ga, lam, gb, y)
        tf = _time(lambda: ops.scan_gelu_fwd(x, gx, ga, lam, gb, y), a.iters, a.warmup, flush)
        tb = _time(lambda: ops.scan_gelu_bwd_into(x, gx, ga, lam, gb, h, y, go, dxy[..., a.D:]), a.iters, a.warmup, flush)
        _emit("scan_gelu_fwd", tf, 6 * es * n, "GB/s", **shape)
        _emit("scan_gelu_bwd", tb, 10 * es * n, "GB/s", **shape)
        _emit("scan_gelu_fwd+bwd", tf + tb, 16 * es * n, "GB/s", **shape)
    elif a.op == "gates":
        M, R, bw = a.B * a.T, a.D, a.bw
        nb = R // bw
        xc, dgx, dga, dxc = (torch.randn(M, R, generator=g, device=dev).bfloat16() for _ in range(4))
        wx, wa = (torch.randn(nb, bw, bw, generator=g, device=dev) / math.sqrt(bw) for _ in range(2))
        packed = ops.gates_pack(wx, wa)
        tf = _time(lambda: ops.gates_fwd(xc, packed, bw), a.iters, a.warmup, flush)
        tb = _time(lambda: ops.gates_bwd_into(xc, dgx, dga, packed, dxc, bw), a.iters, a.warmup, flush)
        ops.check_device_status()
        _emit("gates_fwd", tf, 6 * M * R, "GB/s", M=M, R=R, bw=bw)
        _emit("gates_bwd", tb, 14 * M * R, "GB/s", M=M, R=R, bw=bw)
        # the strided-batch cuBLAS form of the same work
        def bmm_fwd():
            xb = xc.view(M, nb, bw).transpose(0, 1)
            out = torch.empty(2, M, R, dtype=torch.bfloat16, device=dev)
            torch.bmm(xb, wxb, out=out[0].view(M, nb, bw).transpose(0, 1))
            torch.bmm(xb, wab, out=out[1].view(M, nb, bw).transpose(0, 1))
        def bmm_bwd():
            gxb, gab = dgx.view(M, nb, bw).transpose(0, 1), dga.view(M, nb, bw).transpose(0, 1)
            xT = xc.view(M, nb, bw).permute(1, 2, 0)
            torch.bmm(xT, gxb)
            torch.bmm(xT, gab)
            d = dxc.view(M, nb, bw).transpose(0, 1)
            torch.baddbmm(d, gxb, wxb.transpose(1, 2), out=d)
            torch.baddbmm(d, gab, wab.transpose(1, 2), out=d)
        wxb, wab = wx.bfloat16(), wa.bfloat16()
        _emit("gates_fwd_cublas_bmm", _time(bmm_fwd, a.iters, a.warmup, flush), 6 * M * R, "GB/s", M=M, R=R, bw=bw)
        _emit("gates_bwd_cublas_bmm", _time(bmm_bwd, a.iters, a.warmup, flush), 14 * M * R, "GB/s", M=M, R=R, bw=bw)
    elif a.op == "conv1d":
        xy = torch.randn(a.B, a.T, 2 * a.D, generator=g, device=dev).to(dt)
        xv = xy[..., :a.D]  # the strided half the model passes
        go = torch.randn(a.B, a.T, a.D, generator=g, device=dev).to(dt)
        w, b = torch.randn(4, a.D, device=dev) * 0.05, torch.zeros(a.D, device=dev)
        n = a.B * a.T * a.D
        tf = _time(lambda: ops.conv1d_fwd(xv, w, b, dt), a.iters, a.warmup, flush)
        tb = _time(lambda: ops.conv1d_bwd(go, xv, w), a.iters, a.warmup, flush)
        _emit("conv1d_fwd", tf, 2 * es * n, "GB/s", **shape)
        _emit("conv1d_bwd", tb, 3 * es * n, "GB/s", **shape)
    elif a.op == "glue":
        N = a.N if a.N != 8 * 4095 else 8 * 4096
        gu = torch.randn(N, 2 * a.J, generator=g, device=dev).to(dt)  # the projection whose halves are a and b
        av, bv = gu[:, :a.J], gu[:, a.J:]
        go = torch.randn(N, a.J, generator=g, device=dev).to(dt)
        tf = _time(lambda: ops.gelu_mul_fwd(av, bv), a.iters, a.warmup, flush)
        tb = _time(lambda: ops.gelu_mul_bwd(go, av, bv), a.iters, a.warmup, flush)
        _emit("gelu_mul_fwd", tf, 3 * es * N * a.J, "GB/s", N=N, J=a.J, dtype=a.dtype)
        _emit("gelu_mul_bwd", tb, 5 * es * N * a.J, "GB/s", N=N, J=a.J, dtype=a.dtype)
        del gu, av, bv, go
        res = torch.randn(N, a.H, generator=g, device=dev)            # fp32 residual stream
        delta, dy = (torch.randn(N, a.H, generator=g, device=dev).to(dt) for _ in range(2))
        gres = torch.randn(N, a.H, generator=g, device=dev)
        w = torch.ones(a.H, device=dev)
        new_res, y, rstd = ops.add_rms_norm_fwd(res, delta, w, 1e-6, dt)
        tf = _time(lambda: ops.add_rms_norm_fwd(res, delta, w, 1e-6, dt), a.iters, a.warmup, flush)
        tb = _time(lambda: ops.add_rms_norm_bwd(gres, dy, new_res, w, rstd), a.iters, a.warmup, flush)
        _emit("add_rms_norm_fwd", tf, (8 + 2 * es) * N * a.H, "GB/s", N=N, H=a.H, dtype=a.dtype)
        _emit("add_rms_norm_bwd", tb, (12 + 2 * es) * N * a.H, "GB/s", N=N, H=a.H, dtype=a.dtype)
    elif a.op == "linear_ce":
        w = torch.randn(a.V, a.H, generator=g, device=dev) / math.sqrt(a.H)
        act = torch.randn(a.N, a.H, generator=g, device=dev)
        lab = torch.randint(0, a.V, (a.N,), generator=g, device=dev)
        t = _time(lambda: ops.linear_ce(w, act, lab), max(3, a.iters // 4), 2, flush)
        ops.check_device_status()
        _emit("linear_ce", t, 6 * a.N * a.H * a.V, "TFLOP/s", N=a.N, H=a.H, V=a.V)
    elif a.op == "decode_model":
        from .generate import GraphedDecoder
        from .model import HawkModel, hawk_1b_config
        cfg = hawk_1b_config()
        torch.manual_seed(0)
        with torch.device(dev):
            model = HawkModel(cfg, use_cache=True)
        model = model.bfloat16()  # serving precision: weights are read once per token, 2 bytes each
        prompt = torch.randint(1, cfg.vocab_size, (a.B, 16), generator=g, device=dev)
        tok = torch.randint(1, cfg.vocab_size, (a.B, 1), generator=g, device=dev)
        n_params = sum(p.numel() for p in model.parameters())
        for use_graph in (False, True):
            dec = GraphedDecoder(model, a.B, autocast=False, use_graph=use_graph)
            dec.prefill(prompt)
            ms = _time(lambda: dec.step(tok), a.iters, a.warmup)
            print(json.dumps({"kernel": "decode_step_1.35B" + ("_cuda_graph" if use_graph else "_eager"),
                              "ms": round(ms, 4), "tokens_per_s": round(a.B / (ms * 1e-3)),
                              "weight_GBps": round(2 * n_params / (ms * 1e-3) / 1e9, 1), "B": a.B}), flush=True)
    else:
        x, gx, ga = (torch.randn(a.B, a.D, generator=g, device=dev).to(dt) for _ in range(3))
        xy = torch.randn(a.B, 2 * a.D, generator=g, device=dev).to(dt)
        lam = ring_init_(torch.empty(a.D)).to(dev)
        w, b = torch.randn(4, a.D, device=dev) * 0.05, torch.zeros(a.D, device=dev)
        states = [torch.randn(a.B, a.D, generator=g, device=dev).to(dt) for _ in range(a.layers)]
        convs = [torch.randn(a.B, 3, a.D, generator=g, device=dev).to(dt) for _ in range(a.layers)]

        def step():
            for s, c in zip(states, convs):
                ops.decode_conv_step(xy[:, :a.D], c, w, b)
                ops.decode_rglru_step(x, gx, ga, lam, s)
        t = _time(step, a.iters, a.warmup, flush)
        _emit("decode_conv+rglru_step", t / a.layers, 8 * a.B * a.D * es, "GB/s", B=a.B, D=a.D, layers=a.layers,
              dtype=a.dtype)


if __name__ == "__main__":
    main()
