"""Host-side logic of the model shell, on CPU: state-dict contract, wiring against the reference-made
fixture (with the three operators swapped for their oracle statements by the TEST), install()."""
import math
import types

import pytest
import torch
import torch.nn.functional as F

from conftest import load_golden, max_rel
from oracle import model as omodel

import hawk_b200.model as M
from hawk_b200 import install as inst


def _sd(g):
    return {k[3:]: v for k, v in g.items() if k.startswith("sd/")}


def _cfg(g):
    return M.HawkConfig(*[int(v) for v in g["cfg"]])


@pytest.fixture
def oracle_ops(monkeypatch):
    """The product has no CPU path; here the test itself substitutes oracle statements for the kernels."""
    import dp_worker
    dp_worker.patch_ops(monkeypatch.setattr)


def test_state_dict_contract():
    g = load_golden("model_ref.npz")
    model = M.HawkModel(_cfg(g))
    ref = _sd(g)
    mine = model.state_dict()
    assert sorted(mine) == sorted(ref)
    for k in ref:
        assert tuple(mine[k].shape) == tuple(ref[k].shape), k
        assert mine[k].dtype == torch.float32
    model.load_state_dict(ref)  # strict


def test_reference_init_families():
    cfg = M.readme_config()
    torch.manual_seed(0)
    m = M.HawkModel(M.HawkConfig(97, 64, 128, 2, 64, 4, 4))
    assert float(m.lm_head.weight.abs().max()) == 0.0
    for layer in m.layers:
        assert float(layer.recc.resid_proj.weight.abs().max()) == 0.0
        assert float(layer.mlp.resid_proj.weight.abs().max()) == 0.0
        rho = torch.exp(-F.softplus(layer.recc.rg_lru_a_param))
        assert 0.9 - 1e-5 <= float(rho.min()) and float(rho.max()) <= 0.999 + 1e-5
        assert float(layer.recc.conv1d.b.abs().max()) == 0.0
    assert sum(p.numel() for p in M.HawkModel(cfg).parameters()) == 51_945_984
    with torch.device("meta"):
        big = M.HawkModel(M.hawk_1b_config())
    assert sum(p.numel() for p in big.parameters()) == 1_352_108_032


def test_shell_matches_reference_model_fixture(oracle_ops):
    g = load_golden("model_ref.npz")
    model = M.HawkModel(_cfg(g))
    model.load_state_dict(_sd(g))
    loss = model(g["ids"], g["ids"])
    assert abs(float(loss.detach()) - float(g["loss_dezero"])) < 2e-6 * float(g["loss_dezero"])
    loss.backward()
    for k, p in model.named_parameters():
        assert max_rel(p.grad, g["grad/" + k]) < 2e-5, k
    with torch.no_grad():
        assert max_rel(model(g["ids"]), g["logits_dezero"]) < 1e-5


def test_shell_at_reference_init_gives_log_vocab(oracle_ops):
    torch.manual_seed(0)
    cfg = M.HawkConfig(96, 64, 128, 2, 64, 4, 4)
    model = M.HawkModel(cfg)
    ids = torch.randint(1, 96, (2, 17))
    loss = model(ids, ids)
    assert abs(float(loss.detach()) - math.log(96)) < 1e-6
    loss.backward()
    nonzero = [k for k, p in model.named_parameters() if p.grad is not None and float(p.grad.abs().max()) > 0]
    assert nonzero == ["lm_head.weight"]  # every other gradient is exactly zero at the reference init


def test_block_diagonal_linear_matches_einsum():
    torch.manual_seed(1)
    m = M.BlockDiagonalLinear(64, 4)
    with torch.no_grad():
        m.b.normal_()
    x = torch.randn(2, 5, 64)
    assert max_rel(m(x), omodel.block_diag_linear(x, m.w, m.b)) < 1e-6


def test_cache_roll_and_shapes():
    c = M.RNNCache(8, "cpu", 4, batch_size=3, dtype=torch.float32)
    assert c.recc_state.shape == (3, 1, 8) and c.conv_state.shape == (3, 3, 8) and c.current_cache_size == 0
    c.conv_state.copy_(torch.arange(3.0)[None, :, None].expand(3, 3, 8))
    c.update_conv_cache(torch.full((3, 1, 8), 7.0))
    assert c.conv_state[0, :, 0].tolist() == [1.0, 2.0, 7.0]
    c.update_cache(torch.ones(3, 1, 8))
    assert c.current_cache_size == 1


def test_install_rebinds_the_three_names():
    from hawk_b200 import ops
    fake_mod = types.SimpleNamespace(fused_linear_scan=1, fused_cross_entropy=2, Conv1D=3)
    pkg = types.SimpleNamespace(hawk=fake_mod)
    inst.install(pkg)
    assert fake_mod.fused_linear_scan is ops.fused_linear_scan
    assert fake_mod.fused_cross_entropy is ops.fused_cross_entropy and fake_mod.Conv1D is ops.Conv1D
    inst.uninstall(pkg)
    assert (fake_mod.fused_linear_scan, fake_mod.fused_cross_entropy, fake_mod.Conv1D) == (1, 2, 3)


def test_reference_initialiser_names():
    """rnn_param_init / lecun_init under the reference's names and signatures (hawk/external.py:153-168,
    hawk/hawk.py:37-39): exp(-softplus(Lambda)) lands on the [min_rad, max_rad] ring."""
    torch.manual_seed(0)
    lam = M.rnn_param_init(torch.empty(4096), 0.9, 0.999)
    a = torch.exp(-F.softplus(lam.double()))
    assert float(a.min()) >= 0.9 - 1e-6 and float(a.max()) <= 0.999 + 1e-6
    with pytest.raises(NotImplementedError):
        M.rnn_param_init(torch.empty(4), 0.9, 0.999, transform="exp")
    w = torch.empty(512, 256)
    M.lecun_init(w, 256)
    assert abs(float(w.std()) - 1 / math.sqrt(256)) < 0.01 / math.sqrt(256) * 10
