"""Data-parallel step on real GPUs: two NCCL ranks, batch sharded, gradients all-reduced by DDP.  The replicas
stay bit-identical, and losses and first-step gradients equal a single process on the whole batch within the
bf16 bound.  Needs two GPUs (skipped otherwise)."""
import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT, rel_l2

pytestmark = pytest.mark.gpu
WORKER = os.path.join(ROOT, "tests", "dp_gpu_worker.py")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_nccl_ranks_match_single_process(tmp_path):
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT="29641", NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, WORKER, str(tmp_path / "out")], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timeout]"
        outs.append((p.returncode, out))
    assert all(rc == 0 for rc, _ in outs), [o[-800:] for _, o in outs]
    r0, r1 = (torch.load(f"{tmp_path}/out.{r}") for r in range(2))
    for k in r0["params"]:
        assert torch.equal(r0["params"][k], r1["params"][k]), k   # replicas stay bit-identical
        assert torch.equal(r0["grads"][k], r1["grads"][k]), k     # both hold the all-reduced gradient
    assert r0["comm"] and r0["comm"]["buckets"] >= 1 and r0["comm"]["exposed_tail_ms"] >= 0.0

    import dp_gpu_worker as W
    tr = W.make_trainer(torch.device("cuda", 0), 1)
    single = W.run(tr, 0, 1)
    for s in range(3):  # equal token counts per rank: the global loss is the mean of the rank losses
        two = 0.5 * (r0["losses"][s] + r1["losses"][s])
        assert abs(two - single["losses"][s]) <= 2e-2 * abs(single["losses"][s]), (s, two, single["losses"][s])
    for k, gsingle in single["grads"].items():
        assert rel_l2(r0["grads"][k], gsingle) <= 2e-2, (k, rel_l2(r0["grads"][k], gsingle))
