"""Benchmark of the Hawk data-parallel hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1 and per GPU for N > 1): one training step of the ~1.35 B-parameter Hawk model
(vocab 32000, hidden = recurrent = 2048, intermediate 6144, 24 layers, 16 gate blocks, conv width 4)
on B = 8 sequences of T = 4096 uniform-random token ids, bf16 autocast, fused linear cross-entropy,
AdamW update, random (reference) initialisation.  Its RG-LRU scan runs at B=8, T=4096, D=2048 bf16.

One JSON line is printed by rank 0:
  value      whole-job training tokens/s, token ids already resident in HBM;
  e2e        the same through the public API with the step's ids copied from pinned host memory and
             the loss read back every step;
  roofline   the RG-LRU scan forward+backward launches of the step: algorithmic bytes over the mean
             CUDA-event time of those launches INSIDE the timed training steps, against the measured HBM
             copy bandwidth of this pool (MEASURED_PEAKS.json, else the 6650 GB/s fallback);
             `isolated` / `isolated_fused` repeat the measurement outside the step on the plain scan
             (24 B/element) and on the fused entry points (N = 1);
  comm       (N > 1) the gradient all-reduces of one step timed per DDP bucket against the backward pass, and
             every rank's own step time with the all-reduce switched off (what the synchronised step is
             measured against: ranks differ by several ms under the power cap);
             `--grad-comm-dtype bf16` / `--bucket-mb M` change how the gradients are reduced;
  kernels    mean device time and derived rate of each of this library's entry points, from separate
             instrumented steps after the timed regions;
  parity     the check that is free at the reference initialisation: first-step loss = ln 32000 and only
             lm_head.weight has a non-zero gradient;
  configs    (N = 1) the other configurations of the benchmark contract, timed in the same run: the
             scan alone in fp32, one recurrent block, the README model's training step, the long-sequence
             scan and the cached decode step at batch 256;
  reference_gpu  (N = 1) the UNMODIFIED reference package (staged in oracle/_ref by oracle/make_ref.py)
             on the same GPU in the same run: its Triton scan, eager and compiled conv, compiled chunked
             cross-entropy and its HawkModel training step, each beside this library's time;
  cpu_baseline   the CPU oracle of the same model (oracle/model.py) timed on the host cores on a
             bounded sample.

`--impl reference` times that CPU oracle alone (all host threads, same metric and unit).
Launched under torchrun for N > 1 (one rank per GPU, NCCL gradient all-reduce only).
"""
from __future__ import annotations

import argparse
import gc
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "hawk-pytorch_b200"))

import torch  # noqa: E402

B_PER_GPU, SEQ_LEN, VOCAB = 8, 4096, 32000
CPU_SAMPLE_B, CPU_SAMPLE_T = 1, 1024
MODEL = ("vocab 32000, hidden 2048, recurrent 2048, intermediate 6144, 24 layers, 16 gate blocks, conv width 4")
WORKLOAD = f"hawk_1b_train_step: {MODEL}; per-GPU B=8, T=4096; bf16 autocast, fused linear-CE, AdamW"
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one scan forward plus one scan backward
# launch at B=8, T=4096, D=2048 bf16 from one ncu capture of those two kernels: forward 405.2 + 110.5 MB,
# backward 671.1 + 364.9 MB (part of the output is still in L2 when the kernel ends)
SCAN_TRAFFIC_BYTES = 515_724_288 + 1_036_071_168
# the same for the fused entry points (scan + gelu(y)*h), one ncu capture at the same shape: forward 537.0 +
# 239.7 MB (algorithmic 536.9 + 268.4), backward 805.4 + 496.5 MB (algorithmic 805.3 + 536.9)
FUSED_SCAN_TRAFFIC_BYTES = 537_012_224 + 239_708_160 + 805_390_336 + 496_506_880


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", 1400.0)), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return 6650.0, 1400.0, "fallback (6650 GB/s, ~1400 TFLOP/s sustained: earlier measurements on this pool)"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons every 200 ms while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# -------------------------------------------------------------------------------------------------
# CPU arm: the oracle of the same model and step on the host cores
# -------------------------------------------------------------------------------------------------
def cpu_oracle_step_times(steps: int, warmup: int):
    """The CPU oracle of the SAME model and step on a bounded sample; returns the mean seconds of
    (forward + backward, AdamW update) per step."""
    from oracle import model as omodel
    torch.set_num_threads(os.cpu_count() or 1)
    sd = omodel.random_state_dict(VOCAB, 2048, 6144, 24, 2048, 16, 4, seed=0)
    sd = {k: v.requires_grad_(True) for k, v in sd.items()}
    opt = torch.optim.AdamW(list(sd.values()), lr=3e-4, weight_decay=0.1)
    g = torch.Generator().manual_seed(1)
    fb, up = [], []
    for i in range(warmup + steps):
        ids = torch.randint(1, VOCAB, (CPU_SAMPLE_B, CPU_SAMPLE_T), generator=g)
        t0 = time.perf_counter()
        loss = omodel.loss(sd, ids, ids)
        loss.backward()
        t1 = time.perf_counter()
        opt.step()
        opt.zero_grad(set_to_none=True)
        t2 = time.perf_counter()
        if i >= warmup:
            fb.append(t1 - t0)
            up.append(t2 - t1)
    return sum(fb) / len(fb), sum(up) / len(up)


def cpu_baseline_entry(steps: int, warmup: int):
    fb, up = cpu_oracle_step_times(steps, warmup)
    tokens = CPU_SAMPLE_B * CPU_SAMPLE_T
    return {
        "value": tokens / (fb + up), "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
        "sample": (f"B={CPU_SAMPLE_B}, T={CPU_SAMPLE_T} tokens per step of the same 1.35B model on the host cores "
                   f"(fp32 CPU oracle oracle/model.py); {steps} timed steps after {warmup} warm-up; per step "
                   f"{fb:.2f} s forward+backward (scales with tokens) + {up:.2f} s AdamW over 1.35e9 parameters "
                   f"(does not)"),
        "fwd_bwd_s": fb, "adamw_s": up, "fwd_bwd_only_tokens_per_s": tokens / fb,
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return 0
    # every CPU step takes 15-30 s: bound the run to a few minutes whatever K and W were asked for, and
    # report the steps that actually ran
    steps_run, warm_run = min(max(1, args.steps), 2), 1
    cb = cpu_baseline_entry(steps_run, warm_run)
    per_step = cb["fwd_bwd_s"] + cb["adamw_s"]
    line = {
        "impl": "reference", "metric": "hawk_train_tokens_per_sec", "value": cb["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps_run, "warmup": warm_run, "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"hawk_1b_train_step on the host CPU, bounded sample: {MODEL}; B={CPU_SAMPLE_B}, "
                               f"T={CPU_SAMPLE_T} per step; fp32, AdamW",
                   "global_batch": CPU_SAMPLE_B, "seq_len": CPU_SAMPLE_T, "parallelism": "cpu",
                   "requested": {"steps": args.steps, "warmup": args.warmup, "gpus": args.gpus},
                   "note": "reference arm = the reference's algorithm restated for CPU (it ships no CPU scan); the "
                           "sample is smaller than the GPU arm's per-GPU B=8, T=4096 and rank 0 alone runs it"},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# -------------------------------------------------------------------------------------------------
# GPU helpers
# -------------------------------------------------------------------------------------------------
def _median_ms(fn, iters: int, warmup: int, flush=None) -> float:
    """Median device time of one call of fn (CUDA events on the current stream, launches queued back to
    back; `flush`: a buffer larger than L2 rewritten before every timed call)."""
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


def _free():
    gc.collect()
    torch.cuda.empty_cache()


def init_parity(model, loss):
    """Called between the backward and the optimiser update of the FIRST training step.  At the reference
    initialisation lm_head and every resid_proj are zero (hawk/hawk.py:79,128,258), so the first loss is
    ln(vocab) exactly and lm_head.weight is the only parameter with a gradient."""
    nonzero = [k for k, p in model.named_parameters()
               if k != "lm_head.weight" and p.grad is not None and bool((p.grad != 0).any())]
    head = float(model.lm_head.weight.grad.norm())
    err = abs(float(loss) - math.log(VOCAB))
    return {"first_loss": float(loss), "ln_vocab": math.log(VOCAB), "abs_err": err,
            "params_with_nonzero_grad_besides_lm_head": len(nonzero), "lm_head_grad_norm": head,
            "ok": err <= 1e-4 and not nonzero and head > 0}


def other_configs(dev, hbm_peak):
    """The benchmark contract's other configurations, timed on this GPU in this run."""
    import hawk_b200.model as M
    from hawk_b200 import ops, train
    from hawk_b200.generate import GraphedDecoder
    out = {}
    g = torch.Generator(device=dev).manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def scan_case(B, T, D, dt, use_flush):
        es = 2 if dt == torch.bfloat16 else 4
        x, gx, ga, go = (torch.randn(B, T, D, generator=g, device=dev).to(dt) for _ in range(4))
        lam = M.ring_init_(torch.empty(D)).to(dev)
        h = ops.scan_fwd(x, gx, ga, lam)
        f = flush if use_flush else None
        tf = _median_ms(lambda: ops.scan_fwd(x, gx, ga, lam), 20, 5, f)
        tb = _median_ms(lambda: ops.scan_bwd(x, gx, ga, lam, None, None, h, go), 20, 5, f)
        n = B * T * D
        gbs = 12 * es * n / ((tf + tb) * 1e-3) / 1e9
        return {"fwd_ms": tf, "bwd_ms": tb, "GBps": gbs, "frac_of_hbm": gbs / hbm_peak, "algorithmic_bytes": 12 * es * n}

    # config 0: the scan alone, fp32, B=2 T=2048 D=512 (100 MB of traffic: launch- and latency-sized; L2 flushed)
    out["cfg0_scan_B2_T2048_D512_f32"] = scan_case(2, 2048, 512, torch.float32, True)
    # config 4a: long-sequence scan, B=1 T=65536 D=4096 bf16 (6.4 GB of traffic per forward+backward)
    out["cfg4a_scan_B1_T65536_D4096_bf16"] = scan_case(1, 65536, 4096, torch.bfloat16, False)
    _free()

    # config 1: one recurrent block forward+backward, B=8 T=2048 hidden=recurrent=512, 16 gate blocks, bf16 autocast
    cfg1 = M.HawkConfig(VOCAB, 512, 1024, 1, 512, 16, 4)
    torch.manual_seed(0)
    blk = M.Hawk(cfg1).to(dev)
    with torch.no_grad():
        torch.nn.init.normal_(blk.resid_proj.weight, std=1 / math.sqrt(512))
    xin = torch.randn(8, 2048, 512, generator=g, device=dev, requires_grad=True)
    gout = torch.randn(8, 2048, 512, generator=g, device=dev).bfloat16()

    def block_step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y, _ = blk(xin)
        y.backward(gout)
    out["cfg1_block_B8_T2048_R512_bf16"] = {"fwd_bwd_ms": _median_ms(block_step, 20, 5, flush),
                                            "tokens_per_s": None}
    out["cfg1_block_B8_T2048_R512_bf16"]["tokens_per_s"] = 8 * 2048 / (out["cfg1_block_B8_T2048_R512_bf16"]["fwd_bwd_ms"] * 1e-3)
    del blk, xin, gout
    _free()

    # config 2: the README model's training step, B=16 T=2048, bf16 autocast, fused linear-CE, AdamW
    tr = train.Trainer(M.readme_config(), dev, seed=0)
    ids = torch.randint(1, VOCAB, (16, 2048), generator=g, device=dev)
    ms = _median_ms(lambda: tr.step(ids), 10, 3)
    out["cfg2_readme_model_B16_T2048"] = {"ms_per_step": ms, "tokens_per_s": 16 * 2048 / (ms * 1e-3)}
    del tr, ids
    _free()

    # config 4b: one cached token of the 1.35 B model at batch 256 (bf16 weights), whole step as one CUDA graph
    torch.manual_seed(0)
    with torch.device(dev):
        model = M.HawkModel(M.hawk_1b_config(), use_cache=True)
    model = model.bfloat16()
    n_params = sum(p.numel() for p in model.parameters())
    dec = GraphedDecoder(model, 256, autocast=False, use_graph=True)
    dec.prefill(torch.randint(1, VOCAB, (256, 16), generator=g, device=dev))
    tok = torch.randint(1, VOCAB, (256, 1), generator=g, device=dev)
    ms = _median_ms(lambda: dec.step(tok), 20, 5)
    floor_ms = 2 * n_params / (hbm_peak * 1e9) * 1e3
    out["cfg4b_decode_B256_1.35B_bf16"] = {"ms_per_step": ms, "tokens_per_s": 256 / (ms * 1e-3),
                                           "weight_bytes": 2 * n_params, "weight_streaming_floor_ms": floor_ms,
                                           "frac_of_floor": floor_ms / ms}
    del dec, model
    _free()
    return out


def reference_gpu(dev, ours_step_ms: float, with_compiled_model: bool):
    """The staged, unmodified reference package timed on this GPU: each entry holds the reference's time,
    this library's time on the same tensors and `speedup` = theirs / ours.  Nothing here feeds `value`."""
    from oracle import make_ref
    hawk = make_ref.load()
    if hawk is None:
        return {"unavailable": "reference not staged (python oracle/make_ref.py <checkout>)"}
    import hawk_b200.model as M
    from hawk_b200 import ops
    from hawk.external import Conv1D as RefConv
    from hawk.fused_cross_entropy import fused_cross_entropy as ref_ce
    from hawk.scan_fused import sequential_scan_backward, sequential_scan_forward
    out = {"source": "oracle/_ref/hawk (unmodified fattorib/hawk-pytorch, staged by oracle/make_ref.py)",
           "torch": torch.__version__}
    g = torch.Generator(device=dev).manual_seed(11)
    B, T, D = B_PER_GPU, SEQ_LEN, 2048

    def guarded(name, fn):
        try:
            out[name] = fn()
        except Exception as e:  # noqa: BLE001  (a failure of the reference's path on this machine is a result)
            out[name] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
        _free()

    def scan():
        x, gx, ga, go = (torch.randn(B, T, D, generator=g, device=dev).bfloat16() for _ in range(4))
        lam = M.ring_init_(torch.empty(D)).to(dev)
        lam16 = lam.bfloat16()  # what custom_fwd(cast_inputs=bfloat16) hands the kernels, hawk/scan_fused.py:428
        h = sequential_scan_forward(x, gx, ga, lam16)
        tf = _median_ms(lambda: sequential_scan_forward(x, gx, ga, lam16), 5, 2)
        tb = _median_ms(lambda: sequential_scan_backward(x, gx, ga, lam16, h, go), 5, 2)
        ho = ops.scan_fwd(x, gx, ga, lam)
        of = _median_ms(lambda: ops.scan_fwd(x, gx, ga, lam), 20, 5)
        ob = _median_ms(lambda: ops.scan_bwd(x, gx, ga, lam, None, None, ho, go), 20, 5)
        err = float((ho.float() - h.float()).norm() / h.float().norm())
        return {"shape": "B8 T4096 D2048 bf16", "theirs_ms": {"fwd": tf, "bwd": tb}, "ours_ms": {"fwd": of, "bwd": ob},
                "theirs_GBps": 24 * B * T * D / ((tf + tb) * 1e-3) / 1e9, "ours_GBps": 24 * B * T * D / ((of + ob) * 1e-3) / 1e9,
                "speedup": (tf + tb) / (of + ob), "h_rel_l2_ours_vs_theirs": err}

    def conv():
        xy = torch.randn(B, T, 2 * D, generator=g, device=dev).bfloat16().requires_grad_(True)
        go32 = torch.randn(B, T, D, generator=g, device=dev)
        mod = RefConv(width=D, temporal_width=4).to(dev)

        def theirs(m):
            def run():
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    y = m(x=xy[..., :D])  # bf16 strided half in, fp32 out (type promotion, hawk/external.py:88-93)
                y.backward(go32)
                xy.grad = None
            return run
        te = _median_ms(theirs(mod), 5, 2)
        res = {"shape": "B8 T4096 R2048, bf16 strided input, forward+backward through autograd", "theirs_eager_ms": te}
        try:
            tc = _median_ms(theirs(torch.compile(mod)), 5, 3)
            res["theirs_compiled_ms"] = tc
        except Exception as e:  # noqa: BLE001
            res["theirs_compiled_error"] = f"{type(e).__name__}: {str(e)[:200]}"
            tc = None
        w, b = mod.w.detach().clone().requires_grad_(True), mod.b.detach().clone().requires_grad_(True)
        go16 = go32.bfloat16()

        def mine():
            y = ops.temporal_conv1d(xy[..., :D], w, b, out_dtype=torch.bfloat16)
            y.backward(go16)
            xy.grad = None
        om = _median_ms(mine, 20, 5)
        res["ours_ms"] = om
        res["speedup_vs_eager"] = te / om
        if tc:
            res["speedup_vs_compiled"] = tc / om
        return res

    def ce():
        N, H, V = B * (T - 1), 2048, VOCAB
        w = (torch.randn(V, H, generator=g, device=dev) / math.sqrt(H)).requires_grad_(True)
        act = torch.randn(N, H, generator=g, device=dev).requires_grad_(True)
        lab = torch.randint(0, V, (N,), generator=g, device=dev)

        def theirs():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                return ref_ce(w, act, lab)  # gradients are produced inside the forward (fused_cross_entropy.py:55-63)
        wd, ad = w.detach(), act.detach()
        lo = ops.linear_ce(wd, ad, lab)[0]
        ot = _median_ms(lambda: ops.linear_ce(wd, ad, lab), 5, 2)
        ops.check_device_status()
        lt = theirs()
        tt = _median_ms(theirs, 3, 1)
        ot2 = _median_ms(lambda: ops.linear_ce(wd, ad, lab), 5, 2)  # again, after the reference's call
        fl = 6.0 * N * H * V
        return {"shape": "N32760 H2048 V32000, fp32 operands under bf16 autocast, loss + both gradients",
                "theirs_ms": tt, "ours_ms": ot, "ours_ms_after_theirs": ot2, "theirs_TFLOPs": fl / (tt * 1e-3) / 1e12,
                "ours_TFLOPs": fl / (ot * 1e-3) / 1e12, "speedup": tt / ot, "loss_theirs": float(lt.detach()),
                "loss_ours": float(lo)}

    def step(compiled: bool):
        def attempt(bsz):
            torch.manual_seed(0)
            model = hawk.HawkModel(hawk.HawkConfig(VOCAB, 2048, 6144, 24, 2048, 16, 4)).to(dev)
            net = torch.compile(model) if compiled else model
            opt = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.1, fused=True)
            ids = torch.randint(1, VOCAB, (bsz, T), generator=g, device=dev)

            def one():
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    loss = net(ids, ids)
                loss.backward()
                opt.step()
                opt.zero_grad(set_to_none=True)
                return loss
            first = float(one())
            ms = _median_ms(one, 3, 1)
            peak = torch.cuda.max_memory_allocated(dev) / 2**30
            return {"per_gpu_batch": bsz, "ms_per_step": ms, "tokens_per_s": bsz * T / (ms * 1e-3), "first_loss": first,
                    "peak_GiB": peak}
        res = None
        for bsz in (B, B // 2, B // 4):
            try:
                torch.cuda.reset_peak_memory_stats(dev)
                res = attempt(bsz)
                break
            except torch.OutOfMemoryError:
                _free()
        if res is None:
            return {"error": "out of memory at per-GPU batch 8, 4 and 2"}
        res["mode"] = ("torch.compile(model), as the reference README does" if compiled else
                       "eager modules; the reference's cross-entropy wrapper compiles itself (fused_cross_entropy.py:76)")
        ours_tps = B * T / (ours_step_ms * 1e-3)
        res["ours_ms_per_step_B8"] = ours_step_ms
        res["ours_tokens_per_s"] = ours_tps
        res["speedup_tokens_per_s"] = ours_tps / res["tokens_per_s"]
        return res

    guarded("scan_fwd_bwd", scan)
    guarded("conv1d_fwd_bwd", conv)
    guarded("fused_cross_entropy", ce)
    guarded("train_step", lambda: step(False))
    if with_compiled_model:
        guarded("train_step_compiled_model", lambda: step(True))
    return out


# -------------------------------------------------------------------------------------------------
# GPU arm
# -------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist
    import hawk_b200.model as M
    from hawk_b200 import ops, train

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product path has no CPU fallback")
    rank, local_rank, world = train.init_distributed()
    if world != args.gpus:
        raise RuntimeError(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    timeline = train.CommTimeline() if world > 1 else None
    trainer = train.Trainer(M.hawk_1b_config(), dev, seed=0, world_size=world, timeline=timeline,
                            bucket_cap_mb=args.bucket_mb,
                            grad_comm_dtype=torch.bfloat16 if args.grad_comm_dtype == "bf16" else torch.float32)
    g = torch.Generator().manual_seed(1234 + rank)
    n_host = warmup + steps
    host_ids = torch.randint(1, VOCAB, (n_host, B_PER_GPU, SEQ_LEN), generator=g).pin_memory()
    dev_ids = host_ids[:2].to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    scan_names = ops.SCAN_ENTRY_POINTS  # the entry points whose launches are the RG-LRU scan of the step

    # ---- device-resident timing ("value"): only the scan launches are bracketed by events -------
    parity = {}
    trainer.step(dev_ids[0], after_backward=lambda loss: parity.update(init_parity(trainer.model, loss)))
    for i in range(1, warmup):
        trainer.step(dev_ids[i % 2])
    barrier()
    ops.LOG.reset(enabled=True, timed=True, only=scan_names)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        trainer.step(dev_ids[i % 2])
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if sampler else None
    launches = ops.LOG.total_launches()
    scan_ms = {k: ops.LOG.mean_ms(k) for k in ops.LOG.events}
    ops.LOG.reset(enabled=False)
    ops.check_device_status()
    tokens_per_step = world * B_PER_GPU * SEQ_LEN
    value = tokens_per_step * steps / (ms_total * 1e-3)

    # ---- end to end through the public API: pinned host ids in, loss out, every step ------------
    ids_buf = torch.empty(B_PER_GPU, SEQ_LEN, dtype=torch.int64, device=dev)
    barrier()
    e0.record()
    last = 0.0
    for i in range(steps):
        ids_buf.copy_(host_ids[warmup + i], non_blocking=True)
        last = trainer.step(ids_buf).item()
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))
    e2e = tokens_per_step * steps / (ms_e2e * 1e-3)

    # ---- per-entry-point times: two more steps with every C-ABI call bracketed (not part of value) ----
    ops.LOG.reset(enabled=True, timed=True)
    for i in range(2):
        trainer.step(dev_ids[i % 2])
    barrier()
    kernel_ms = {k: ops.LOG.mean_ms(k) for k in ops.LOG.events}
    ops.LOG.reset(enabled=False)
    comm = timeline.summary() if timeline is not None else None  # the gradient all-reduces of the last step

    # ---- N > 1: every rank's own step with the all-reduce switched off (last thing the replicas do together:
    # they diverge from here).  Tells rank skew and DDP's own overhead apart from communication. ----
    if world > 1:
        trainer.step(dev_ids[0], sync_gradients=False)
        torch.cuda.synchronize()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for i in range(3):
            trainer.step(dev_ids[i % 2], sync_gradients=False)
        c1.record()
        torch.cuda.synchronize()
        mine = torch.tensor([c0.elapsed_time(c1) / 3], device=dev, dtype=torch.float64)
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        per_rank = [float(t.item()) for t in every]
        if comm is None:
            comm = {}
        comm["compute_only_ms_per_rank"] = [round(v, 2) for v in per_rank]
        comm["compute_only_what"] = ("ms per step of each rank with the gradient all-reduce switched off (3 steps after "
                                     "everything else was measured): the synchronised step cannot be faster than the "
                                     "slowest of these")

    if rank != 0:
        return 0

    hbm_peak, tensor_peak, peak_src = measured_peaks()
    n_elem = B_PER_GPU * SEQ_LEN * 2048

    # the plain scan kernels alone, back to back on resident tensors (no GEMMs around them drawing power)
    isolated = None
    if world == 1:
        del ids_buf
        g2 = torch.Generator(device=dev).manual_seed(7)
        xs = [torch.randn(B_PER_GPU, SEQ_LEN, 2048, generator=g2, device=dev).bfloat16() for _ in range(4)]
        lam = trainer.model.layers[0].recc.rg_lru_a_param.detach().float()
        gb = 0.1 * torch.randn(2, 2048, generator=g2, device=dev)  # gate biases, as the training step passes them
        h = ops.scan_fwd(xs[0], xs[1], xs[2], lam, None, gb)
        for _ in range(3):
            ops.scan_fwd(xs[0], xs[1], xs[2], lam, None, gb)
            ops.scan_bwd(xs[0], xs[1], xs[2], lam, None, gb, h, xs[3])
        torch.cuda.synchronize()
        time.sleep(3.0)  # let the board leave the power-capped state of the training loop: a burst figure
        isolated = {"fwd_ms": _median_ms(lambda: ops.scan_fwd(xs[0], xs[1], xs[2], lam, None, gb), 20, 5),
                    "bwd_ms": _median_ms(lambda: ops.scan_bwd(xs[0], xs[1], xs[2], lam, None, gb, h, xs[3]), 20, 5)}
        # the fused entry points the step launches, alone in the same state
        xy = torch.randn(B_PER_GPU, SEQ_LEN, 4096, generator=g2, device=dev).bfloat16()
        dxy = torch.empty_like(xy)
        hh, _ = ops.scan_gelu_fwd(xs[0], xs[1], xs[2], lam, gb, xy[..., 2048:])
        isolated["fused_fwd_ms"] = _median_ms(lambda: ops.scan_gelu_fwd(xs[0], xs[1], xs[2], lam, gb, xy[..., 2048:]), 20, 5)
        isolated["fused_bwd_ms"] = _median_ms(
            lambda: ops.scan_gelu_bwd_into(xs[0], xs[1], xs[2], lam, gb, hh, xy[..., 2048:], xs[3], dxy[..., 2048:]), 20, 5)
        del xs, h, hh, xy, dxy

    # bytes each launch must move: [bytes per element forward, backward] of the entry points the step uses
    fwd_name, bwd_name = scan_names
    bpe_f, bpe_b = ops.SCAN_BYTES_PER_ELEMENT[fwd_name], ops.SCAN_BYTES_PER_ELEMENT[bwd_name]
    roofline = {"bound": "hbm", "achieved": None, "peak": hbm_peak, "unit": "GB/s", "frac": None,
                "traffic": SCAN_TRAFFIC_BYTES if (bpe_f, bpe_b) == (8, 16) else FUSED_SCAN_TRAFFIC_BYTES,
                "kernel": f"{fwd_name} + {bwd_name}, B=8 T=4096 D=2048 bf16, inside the training step",
                "algorithmic_bytes": (bpe_f + bpe_b) * n_elem, "bytes_per_element": {"fwd": bpe_f, "bwd": bpe_b},
                "peak_source": peak_src}
    if scan_ms.get(fwd_name) and scan_ms.get(bwd_name):
        t = (scan_ms[fwd_name] + scan_ms[bwd_name]) * 1e-3
        roofline["achieved"] = (bpe_f + bpe_b) * n_elem / t / 1e9
        roofline["frac"] = roofline["achieved"] / hbm_peak
        roofline["launch_ms"] = {"fwd": scan_ms[fwd_name], "bwd": scan_ms[bwd_name]}
    if isolated:
        t = (isolated["fwd_ms"] + isolated["bwd_ms"]) * 1e-3
        roofline["isolated"] = {"achieved": 24 * n_elem / t / 1e9, "frac": 24 * n_elem / t / 1e9 / hbm_peak,
                                "launch_ms": {"fwd": isolated["fwd_ms"], "bwd": isolated["bwd_ms"]},
                                "note": "scan_fwd + scan_bwd (24 B/element), same shape, median of 20 back-to-back "
                                        "launches each outside the step, after 3 s idle (burst clocks)"}
        tf = (isolated["fused_fwd_ms"] + isolated["fused_bwd_ms"]) * 1e-3
        roofline["isolated_fused"] = {"achieved": 32 * n_elem / tf / 1e9, "frac": 32 * n_elem / tf / 1e9 / hbm_peak,
                                      "launch_ms": {"fwd": isolated["fused_fwd_ms"], "bwd": isolated["fused_bwd_ms"]},
                                      "note": "scan_gelu_fwd + scan_gelu_bwd (32 B/element), measured the same way"}
    kernels = {}
    n_ce = B_PER_GPU * (SEQ_LEN - 1)
    rates = {"conv1d_fwd": (4 * n_elem, "GB/s"), "conv1d_bwd": (6 * n_elem, "GB/s"),
             "linear_ce": (6 * n_ce * 2048 * VOCAB, "TFLOP/s")}
    for k, bpe in ops.SCAN_BYTES_PER_ELEMENT.items():
        rates[k] = (bpe * n_elem, "GB/s")
    for k, bpe in getattr(ops, "GATE_BYTES_PER_ELEMENT", {}).items():
        rates[k] = (bpe * n_elem, "GB/s")
    for k, ms in kernel_ms.items():
        entry = {"mean_ms": ms}
        if k in rates and ms:
            work, unit = rates[k]
            entry["rate"] = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
            entry["unit"] = unit
            entry["frac_of_peak"] = entry["rate"] / (hbm_peak if unit == "GB/s" else tensor_peak)
        kernels[k] = entry

    line = {
        "metric": "hawk_train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms_total / steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": B_PER_GPU * world, "seq_len": SEQ_LEN,
                   "parallelism": f"dp{world}",
                   "l2": "no flush needed: each step streams > 100 GB of activations, far beyond the 126 MB L2"},
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": B_PER_GPU * SEQ_LEN * 8,
                "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e / steps, "last_loss": last},
        "gpu_launches": launches, "roofline": roofline, "kernels": kernels, "clocks": clocks, "parity": parity,
    }
    if world > 1:
        line["config"]["grad_all_reduce"] = {"dtype": args.grad_comm_dtype, "bucket_mb": args.bucket_mb}
    if comm is not None:
        comm["what"] = ("gradient all-reduce per DDP bucket in one step on rank 0: time from the bucket being ready on the "
                        "compute stream to its all-reduce being done, and how far the last all-reduce ran past the moment "
                        "the last bucket was ready (communication the backward pass did not hide)")
        line["comm"] = comm

    if world == 1:
        del trainer, dev_ids
        _free()
        if not args.no_configs:
            try:
                line["configs"] = other_configs(dev, hbm_peak)
            except Exception as e:  # noqa: BLE001
                line["configs"] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
            _free()
        if not args.no_reference_gpu:
            line["reference_gpu"] = reference_gpu(dev, ms_total / steps, args.reference_gpu_compile)
            _free()
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_entry(steps=2, warmup=1)
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true",
                    help="skip the CPU-oracle leg (e.g. when the command runs under a profiler)")
    ap.add_argument("--no-configs", action="store_true", help="skip the other configurations (N = 1 only)")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip the reference-on-GPU block (N = 1 only)")
    ap.add_argument("--grad-comm-dtype", default="f32", choices=["f32", "bf16"],
                    help="N > 1: dtype of the gradient all-reduce (bf16 halves the NVLink bytes)")
    ap.add_argument("--bucket-mb", type=int, default=256,
                    help="N > 1: DDP bucket size; larger than the 5.4 GB of gradients = one all-reduce after the backward")
    ap.add_argument("--reference-gpu-compile", action="store_true",
                    help="also time the reference training step with torch.compile(model) (minutes of compilation)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)
    rc = run_ours(args)
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()
    return rc


if __name__ == "__main__":
    sys.exit(main())
