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
  roofline   the RG-LRU scan forward+backward: algorithmic bytes (24 B/element in bf16) over the mean
             CUDA-event time of the scan launches INSIDE the timed training steps, against the
             measured HBM copy bandwidth of this pool (MEASURED_PEAKS.json, else the 6650 GB/s fallback);
             `isolated` repeats the measurement on the same kernels outside the step (N = 1 only);
  kernels    mean device time and derived rate of each of this library's entry points in the same steps;
  cpu_baseline   the CPU oracle of the same model (oracle/model.py) timed on the host cores on a
             bounded sample (B=1, T=128 per step).

`--impl reference` times that CPU oracle alone (all host threads, same metric and config).
Launched under torchrun for N > 1 (one rank per GPU, NCCL gradient all-reduce only).
"""
from __future__ import annotations

import argparse
import json
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
CPU_SAMPLE_B, CPU_SAMPLE_T = 1, 128
WORKLOAD = ("hawk_1b_train_step: vocab 32000, hidden 2048, recurrent 2048, intermediate 6144, 24 layers, "
            "16 gate blocks, conv width 4; per-GPU B=8, T=4096; bf16 autocast, fused linear-CE, AdamW")
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one scan forward plus one scan backward
# launch at B=8, T=4096, D=2048 bf16, from the ncu capture summarised in profiles/scan_B8_D2048_bf16.md
# (forward 405.2 + 110.5 MB, backward 671.1 + 364.9 MB; part of the output is still in L2 at kernel end)
SCAN_TRAFFIC_BYTES = 515_724_288 + 1_036_071_168


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6650 GB/s, earlier measurement on this pool)"


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


def cpu_oracle_tokens_per_sec(steps: int, warmup: int):
    """The CPU oracle of the SAME model and step (forward, backward, AdamW) on a bounded sample."""
    from oracle import model as omodel
    torch.set_num_threads(os.cpu_count() or 1)
    sd = omodel.random_state_dict(VOCAB, 2048, 6144, 24, 2048, 16, 4, seed=0)
    sd = {k: v.requires_grad_(True) for k, v in sd.items()}
    opt = torch.optim.AdamW(list(sd.values()), lr=3e-4, weight_decay=0.1)
    g = torch.Generator().manual_seed(1)
    times = []
    for i in range(warmup + steps):
        ids = torch.randint(1, VOCAB, (CPU_SAMPLE_B, CPU_SAMPLE_T), generator=g)
        t0 = time.perf_counter()
        loss = omodel.loss(sd, ids, ids)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    per_step = sum(times) / len(times)
    return CPU_SAMPLE_B * CPU_SAMPLE_T / per_step, per_step


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return 0
    steps, warmup = max(1, args.steps), max(1, args.warmup)
    # every CPU step is ~seconds: bound the run to a few minutes whatever K and W were asked for
    steps_run, warm_run = min(steps, 8), min(warmup, 1)
    tps, per_step = cpu_oracle_tokens_per_sec(steps_run, warm_run)
    cores = torch.get_num_threads()
    sample = (f"B={CPU_SAMPLE_B}, T={CPU_SAMPLE_T} tokens per step of the same 1.35B model (fp32, CPU oracle "
              f"oracle/model.py: forward, backward, AdamW); {steps_run} timed steps after {warm_run} warm-up")
    line = {
        "impl": "reference", "metric": "hawk_train_tokens_per_sec", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": B_PER_GPU * args.gpus, "seq_len": SEQ_LEN,
                   "parallelism": f"dp{args.gpus}", "note": "reference arm = the reference's algorithm restated "
                   "for CPU (it ships no CPU scan); bounded sample, see cpu_baseline.sample"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


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

    trainer = train.Trainer(M.hawk_1b_config(), dev, seed=0, world_size=world)
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

    # ---- device-resident timing ("value") ------------------------------------------------------
    for i in range(warmup):
        trainer.step(dev_ids[i % 2])
    barrier()
    ops.LOG.reset(enabled=True, timed=True)
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
    kernel_ms = {k: ops.LOG.mean_ms(k) for k in ops.LOG.events}
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

    if rank != 0:
        return 0

    # the same two kernels alone, back to back on resident tensors (no GEMMs around them drawing power)
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
        ops.LOG.reset(enabled=True, timed=True)
        for _ in range(20):
            ops.scan_fwd(xs[0], xs[1], xs[2], lam, None, gb)
        for _ in range(20):
            ops.scan_bwd(xs[0], xs[1], xs[2], lam, None, gb, h, xs[3])
        torch.cuda.synchronize()
        isolated = {"fwd_ms": ops.LOG.mean_ms("scan_fwd"), "bwd_ms": ops.LOG.mean_ms("scan_bwd")}
        ops.LOG.reset(enabled=False)
        del xs, h

    n_elem = B_PER_GPU * SEQ_LEN * 2048
    peak, peak_src = measured_hbm_peak()
    roofline = {"bound": "hbm", "achieved": None, "peak": peak, "unit": "GB/s", "frac": None,
                "traffic": SCAN_TRAFFIC_BYTES, "kernel": "scan_fwd_kernel + scan_bwd_kernel, B=8 T=4096 D=2048 bf16",
                "algorithmic_bytes": 24 * n_elem, "peak_source": peak_src}
    if kernel_ms.get("scan_fwd") and kernel_ms.get("scan_bwd"):
        t = (kernel_ms["scan_fwd"] + kernel_ms["scan_bwd"]) * 1e-3
        roofline["achieved"] = 24 * n_elem / t / 1e9
        roofline["frac"] = roofline["achieved"] / peak
        roofline["launch_ms"] = {"fwd": kernel_ms["scan_fwd"], "bwd": kernel_ms["scan_bwd"]}
    if isolated:
        t = (isolated["fwd_ms"] + isolated["bwd_ms"]) * 1e-3
        roofline["isolated"] = {"achieved": 24 * n_elem / t / 1e9, "frac": 24 * n_elem / t / 1e9 / peak,
                                "launch_ms": {"fwd": isolated["fwd_ms"], "bwd": isolated["bwd_ms"]},
                                "note": "same kernels and shape, 20 back-to-back launches each outside the step, after 3 s idle (burst clocks)"}
    kernels = {}
    n_ce = B_PER_GPU * (SEQ_LEN - 1)
    rates = {"scan_fwd": (8 * n_elem, "GB/s"), "scan_bwd": (16 * n_elem, "GB/s"), "conv1d_fwd": (4 * n_elem, "GB/s"),
             "conv1d_bwd": (6 * n_elem, "GB/s"), "linear_ce": (6 * n_ce * 2048 * VOCAB, "TFLOP/s")}
    for k, ms in kernel_ms.items():
        entry = {"mean_ms": ms}
        if k in rates and ms:
            work, unit = rates[k]
            entry["rate"] = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
            entry["unit"] = unit
        kernels[k] = entry

    run_cpu = world == 1 and not args.no_cpu_baseline
    cpu_tps, cpu_step = cpu_oracle_tokens_per_sec(steps=2, warmup=1) if run_cpu else (None, None)
    line = {
        "metric": "hawk_train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms_total / steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": B_PER_GPU * world, "seq_len": SEQ_LEN,
                   "parallelism": f"dp{world}",
                   "l2": "no flush needed: each step streams > 100 GB of activations, far beyond the 126 MB L2"},
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": B_PER_GPU * SEQ_LEN * 8,
                "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e / steps, "last_loss": last},
        "gpu_launches": launches, "roofline": roofline, "kernels": kernels, "clocks": clocks,
    }
    if cpu_tps is not None:
        line["cpu_baseline"] = {
            "value": cpu_tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": (f"B={CPU_SAMPLE_B}, T={CPU_SAMPLE_T} tokens per step of the same 1.35B model on the host "
                       f"cores (fp32 CPU oracle: forward, backward, AdamW), 2 timed steps after 1 warm-up, "
                       f"{cpu_step:.2f} s per step")}
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
