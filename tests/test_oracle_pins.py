"""Pins the CPU oracle to outputs of the unmodified reference (tests/golden/*.npz,
made by tests/golden/make_golden.py) and to closed-form / autograd checks.  CPU only."""
import math

import pytest
import torch

from conftest import load_golden, max_rel, rel_l2
from oracle import conv1d as oconv
from oracle import linear_ce as oce
from oracle import model as omodel
from oracle import scan as oscan


def _assert_same_up_to_ulp_straddles(got, want, max_frac=0.01):
    """Equal bit for bit, except where a last-bit difference in an fp32 intermediate (torch's
    exp/sigmoid vs the interpreter's numpy ones) falls across a bf16 truncation boundary, or is
    amplified by the cancellation in 1 - a^2 when a gate saturates.  Such elements must stay
    rare and small against the tensor's scale."""
    bad = got != want
    assert float(bad.float().mean()) <= max_frac
    assert max_rel(got, want) < 2.0**-7  # at most one bf16 ulp of the largest element


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_scan_oracle_equals_reference_triton_kernels(tag):
    """With the interpreter's truncating bf16 stores emulated, the restatement reproduces the
    reference kernels' h, dx, dgx, dga bit for bit (up to rare one-ulp straddles, see above);
    dlam differs only by summation rounding."""
    g = load_golden("scan_triton_interp.npz")
    x, gx, ga, go, lam = (g[f"{tag}_{k}"] for k in ("x", "gx", "ga", "go", "lam"))
    h = oscan.rglru_scan_fwd(x, gx, ga, lam, store="bf16_trunc")
    _assert_same_up_to_ulp_straddles(h, g[f"{tag}_h"])
    dx, dgx, dga, dlam = oscan.rglru_scan_bwd(x, gx, ga, lam, g[f"{tag}_h"], go, store="bf16_trunc")
    _assert_same_up_to_ulp_straddles(dx, g[f"{tag}_dx"])
    _assert_same_up_to_ulp_straddles(dgx, g[f"{tag}_dgx"])
    _assert_same_up_to_ulp_straddles(dga, g[f"{tag}_dga"])
    assert max_rel(dlam, g[f"{tag}_dlam"]) < 2e-6
    # the un-rounded fp32 restatement (what the CUDA kernels are held to) sits within the
    # truncation error of the reference's bf16-valued outputs
    assert max_rel(oscan.rglru_scan_fwd(x, gx, ga, lam), g[f"{tag}_h"]) < 2.0**-7


def test_scan_oracle_closed_form():
    lam = oscan.rnn_param_ring(64, generator=torch.Generator().manual_seed(3)).double()
    T = 300
    ones = torch.ones(1, T, 64, dtype=torch.float64)
    zeros = torch.zeros_like(ones)
    h = oscan.rglru_scan_fwd(ones, zeros, zeros, lam, compute=torch.float64)
    assert max_rel(h, oscan.closed_form_kat(lam, T)) < 1e-13


def test_scan_oracle_backward_equals_autograd():
    g = torch.Generator().manual_seed(4)
    B, T, D = 2, 33, 64
    x, gx, ga, go = (torch.randn(B, T, D, generator=g, dtype=torch.float64) for _ in range(4))
    lam = oscan.rnn_param_ring(D, generator=g).double()
    h = oscan.rglru_scan_fwd(x, gx, ga, lam, compute=torch.float64)
    got = oscan.rglru_scan_bwd(x, gx, ga, lam, h, go, compute=torch.float64)
    ref = oscan.rglru_scan_autograd(x, gx, ga, lam, go)
    assert max_rel(h, ref[0]) < 1e-13
    for a, b in zip(got, ref[1:]):
        assert max_rel(a, b) < 1e-11


def test_scan_oracle_fp32_close_to_fp64():
    g = torch.Generator().manual_seed(5)
    B, T, D = 2, 512, 64
    x, gx, ga, go = (torch.randn(B, T, D, generator=g) for _ in range(4))
    lam = oscan.rnn_param_ring(D, generator=g)
    h32 = oscan.rglru_scan_fwd(x, gx, ga, lam)
    h64 = oscan.rglru_scan_fwd(x, gx, ga, lam, compute=torch.float64)
    assert rel_l2(h32, h64) < 1e-6


def test_ring_init_range():
    lam = oscan.rnn_param_ring(4096, generator=torch.Generator().manual_seed(0))
    rho = torch.exp(-torch.nn.functional.softplus(lam))
    assert 0.9 - 1e-6 <= float(rho.min()) and float(rho.max()) <= 0.999 + 1e-6


def test_conv_oracle_equals_reference_module():
    g = load_golden("conv1d_ref.npz")
    y = oconv.conv1d_fwd(g["x"], g["w"], g["b"])
    assert max_rel(y, g["y"]) < 1e-6
    dx, dw, db = oconv.conv1d_bwd(g["x"], g["w"], g["go"])
    assert max_rel(dx, g["dx"]) < 1e-6
    assert max_rel(dw, g["dw"]) < 1e-6
    assert max_rel(db, g["db"]) < 1e-6
    assert max_rel(oconv.conv1d_fwd(g["short_x"], g["w"], g["b"]), g["short_y"]) < 1e-6


def test_ce_oracle_equals_reference_function():
    g = load_golden("linear_ce_ref.npz")
    loss, dw, dact = oce.linear_ce_fwd_bwd(g["w"], g["act"], g["labels"])
    up = float(g["upstream"])
    assert abs(float(loss) - float(g["loss"])) < 1e-6 * abs(float(g["loss"]))
    assert max_rel(up * dw, g["dw"]) < 1e-6
    assert max_rel(up * dact, g["dact"]) < 1e-6
    l64, dw64, da64 = oce.linear_ce_direct(g["w"], g["act"], g["labels"])
    assert abs(float(loss) - float(l64)) < 1e-6
    assert max_rel(dw, dw64) < 1e-5 and max_rel(dact, da64) < 1e-5


def test_ce_oracle_bf16_emulation_is_close():
    g = load_golden("linear_ce_ref.npz")
    l32, dw32, da32 = oce.linear_ce_fwd_bwd(g["w"], g["act"], g["labels"])
    l16, dw16, da16 = oce.linear_ce_fwd_bwd(g["w"], g["act"], g["labels"], autocast_bf16=True)
    assert abs(float(l16) - float(l32)) < 2e-2 * float(l32)
    assert rel_l2(dw16, dw32) < 2e-2 and rel_l2(da16, da32) < 2e-2


def _model_sd(g):
    return {k[3:]: v for k, v in g.items() if k.startswith("sd/")}


def test_model_oracle_equals_reference_model():
    g = load_golden("model_ref.npz")
    V = int(g["cfg"][0])
    assert abs(float(g["loss_init"]) - math.log(V)) < 1e-6  # zero lm_head => uniform logits
    sd = {k: v.clone().requires_grad_(True) for k, v in _model_sd(g).items()}
    loss = omodel.loss(sd, g["ids"], g["ids"])
    assert abs(float(loss.detach()) - float(g["loss_dezero"])) < 2e-6 * float(g["loss_dezero"])
    loss.backward()
    for k, p in sd.items():
        assert max_rel(p.grad, g["grad/" + k]) < 2e-5, k
    with torch.no_grad():
        assert max_rel(omodel.logits(sd, g["ids"]), g["logits_dezero"]) < 1e-5


def test_decode_oracle_equals_reference_cached_path():
    sd = _model_sd(load_golden("model_ref.npz"))
    g = load_golden("decode_ref.npz")
    ids = g["ids"]
    with torch.no_grad():
        logits, caches = omodel.prefill(sd, ids[:, :5])
        assert max_rel(logits, g["prefill_logits"]) < 1e-5
        for s in range(3):
            logits, caches = omodel.decode_step(sd, ids[:, 5 + s : 6 + s], caches)
            assert max_rel(logits, g[f"step{s}_logits"]) < 1e-5, s
        assert torch.equal(caches[0]["recc"].float()[:, None], g["final_recc_state0"])
        assert max_rel(caches[0]["conv"], g["final_conv_state0"]) < 1e-6
        # cached steps reproduce the full-sequence forward (bf16 state rounding aside)
        full = omodel.logits(sd, ids)
        assert max_rel(logits[:, 0], full[:, -1]) < 2e-2
