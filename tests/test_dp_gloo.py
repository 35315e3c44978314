"""Data-parallel harness on CPU: two gloo ranks, batch sharded, gradients all-reduced.  Replicas stay
identical and equal a single process trained on the whole batch; a rank that dies is detected."""
import os
import subprocess
import sys

import torch

from conftest import ROOT, max_rel

WORKER = os.path.join(ROOT, "tests", "dp_worker.py")


def _launch(tmp_path, world, port, extra=(), timeout=240):
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2", GLOO_SOCKET_IFNAME="lo")
        procs.append(subprocess.Popen([sys.executable, WORKER, str(tmp_path / "out"), *extra], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timeout]"
        outs.append((p.returncode, out))
    return outs


def test_two_ranks_match_single_process(tmp_path, monkeypatch):
    outs = _launch(tmp_path, 2, 29631)
    assert all(rc == 0 for rc, _ in outs), outs
    r0, r1 = (torch.load(f"{tmp_path}/out.{r}") for r in range(2))
    for k in r0["params"]:
        assert torch.equal(r0["params"][k], r1["params"][k]), k  # replicas stay bit-identical

    import dp_worker as W
    W.patch_ops(monkeypatch.setattr)  # the same substitution the workers make, undone after this test
    tr = W.make_trainer(1)
    single = [float(tr.step(W.data(s))) for s in range(3)]
    # the global loss is the mean of the two rank losses (equal token counts per rank)
    for s in range(3):
        assert abs(0.5 * (r0["losses"][s] + r1["losses"][s]) - single[s]) < 1e-5 * abs(single[s])
    for k, v in tr.model.state_dict().items():
        assert max_rel(r0["params"][k], v) < 1e-4, k


def test_dead_rank_is_detected_not_hung(tmp_path):
    """Rank 1 exits between steps; rank 0's next collective must end with an error (gloo reports the
    closed connection), well inside the timeout."""
    outs = _launch(tmp_path, 2, 29633, extra=("1",), timeout=180)
    assert outs[1][0] == 17
    assert outs[0][0] != 0 and "[timeout]" not in outs[0][1], outs[0][1][-500:]


def test_step_without_gradient_sync_is_local(tmp_path):
    """`Trainer.step(sync_gradients=False)` (the benchmark's per-rank compute-only measurement): no collective
    runs, each rank applies its own gradients, so replicas that were bit-identical differ afterwards."""
    outs = _launch(tmp_path, 2, 29635, extra=("-1", "unsynced"))
    assert all(rc == 0 for rc, _ in outs), outs
    t0, t1 = (torch.load(f"{tmp_path}/out.tail.{r}") for r in range(2))
    assert all(torch.equal(t0["synced"][k], t1["synced"][k]) for k in t0["synced"])
    moved = [k for k in t0["after"] if not torch.equal(t0["after"][k], t0["synced"][k])]
    differ = [k for k in t0["after"] if not torch.equal(t0["after"][k], t1["after"][k])]
    assert moved and differ  # the step was taken, with rank-local gradients
