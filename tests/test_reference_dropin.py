"""Drop-in check against the real reference package, staged by `python oracle/make_ref.py` into
oracle/_ref (skipped when absent): install() rebinds the three operator names inside hawk/hawk.py and
the reference's own HawkModel then runs through them with its own call conventions (keyword `x=` for
the conv, positional scan arguments, `.view`-ed cross-entropy inputs) and reproduces the fixture.
CPU only: the operators are substituted by their oracle statements BEFORE install() binds them, so
this exercises names, signatures and parameter layout, not the kernels."""
import os
import sys

import pytest
import torch
import torch.nn.functional as F

from conftest import load_golden, max_rel
from oracle import make_ref
from oracle import model as omodel


@pytest.mark.skipif(not make_ref.available(), reason="reference not staged (python oracle/make_ref.py <checkout>)")
def test_reference_model_runs_on_the_rebound_operators(monkeypatch):
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    hawk = make_ref.load()  # the reference package
    from hawk_b200 import install, ops

    class OracleConv1D(ops.Conv1D):  # same parameters and constructor; CPU statement of the forward
        def forward(self, x):
            return omodel.conv1d(x, self.w, self.b)

    monkeypatch.setattr(ops, "fused_linear_scan", lambda x, gx, ga, lam: omodel.scan(x, gx, ga, lam))
    monkeypatch.setattr(ops, "fused_cross_entropy", lambda w, a, l: F.cross_entropy(F.linear(a, w), l))
    monkeypatch.setattr(ops, "Conv1D", OracleConv1D)
    original = (hawk.hawk.fused_linear_scan, hawk.hawk.fused_cross_entropy, hawk.hawk.Conv1D)
    install.install(hawk)
    try:
        assert hawk.hawk.Conv1D is OracleConv1D and hawk.hawk.fused_linear_scan is ops.fused_linear_scan
        g = load_golden("model_ref.npz")
        cfg = hawk.HawkConfig(*[int(v) for v in g["cfg"]])
        model = hawk.HawkModel(cfg)
        sd = {k[3:]: v for k, v in g.items() if k.startswith("sd/")}
        model.load_state_dict(sd)  # the conv module keeps the reference's parameter names
        loss = model(g["ids"], g["ids"])
        assert abs(float(loss.detach()) - float(g["loss_dezero"])) < 2e-6 * float(g["loss_dezero"])
        loss.backward()
        for k, p in model.named_parameters():
            assert max_rel(p.grad, g["grad/" + k]) < 2e-5, k
    finally:
        install.uninstall(hawk)
        assert (hawk.hawk.fused_linear_scan, hawk.hawk.fused_cross_entropy, hawk.hawk.Conv1D) == original
        for m in [m for m in sys.modules if m == "hawk" or m.startswith("hawk.")]:
            del sys.modules[m]
