"""Parity of the CUDA RG-LRU scan (through the C ABI) with the CPU oracle.

Tolerances (norm-wise; element-wise relative error is meaningless at zero crossings):
  fp32 storage : rel-L2 and max-abs/max-abs <= 1e-5 against the fp64 oracle;
  bf16 storage : <= 2e-2 against the fp64 oracle run on the same bf16-rounded inputs.
"""
import pytest
import torch

from conftest import load_golden, max_rel, rel_l2
from oracle import scan as oscan

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
BF16_TOL = 2e-2


def _inputs(B, T, D, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    x, gx, ga, go = (scale * torch.randn(B, T, D, generator=g) for _ in range(4))
    lam = oscan.rnn_param_ring(D, generator=g)
    if dtype != torch.float32:  # the oracle sees exactly the values the kernel sees
        x, gx, ga, go = (t.to(dtype).float() for t in (x, gx, ga, go))
    return x, gx, ga, go, lam


def _run_gpu(x, gx, ga, go, lam, dtype, h0=None):
    from hawk_b200 import fused_linear_scan
    dev = "cuda:0"
    xs = [t.to(dev, dtype).requires_grad_(True) for t in (x, gx, ga)]
    lam_d = lam.to(dev).requires_grad_(True)
    h0_d = None if h0 is None else h0.to(dev).requires_grad_(True)
    h = fused_linear_scan(*xs, lam_d, h0=h0_d)
    assert h.dtype == dtype and h.shape == x.shape
    h.backward(go.to(dev, dtype))
    outs = [h.detach()] + [t.grad for t in xs] + [lam_d.grad]
    if h0 is not None:
        outs.append(h0_d.grad)
    return [o.float().cpu() for o in outs]


def _oracle(x, gx, ga, go, lam, h_stored):
    h = oscan.rglru_scan_fwd(x, gx, ga, lam, compute=torch.float64)
    # the backward reads the h that was actually stored (rounded), as the reference does
    grads = oscan.rglru_scan_bwd(x, gx, ga, lam, h_stored.double(), go, compute=torch.float64)
    return (h,) + grads


def _check(got, want, tol, names=("h", "dx", "dgx", "dga", "dlam")):
    for n, a, b in zip(names, got, want):
        assert rel_l2(a, b) <= tol, (n, rel_l2(a, b))
        assert max_rel(a, b) <= tol, (n, max_rel(a, b))


SHAPES = [(1, 1, 64), (1, 2, 64), (2, 3, 128), (2, 31, 64), (2, 32, 64), (2, 33, 64), (1, 63, 128), (1, 64, 128),
          (1, 65, 128), (3, 257, 192), (2, 2048, 512), (1, 1000, 4096)]


@pytest.mark.parametrize("B,T,D", SHAPES)
def test_scan_fp32_matches_oracle(B, T, D):
    x, gx, ga, go, lam = _inputs(B, T, D, seed=B * 1000 + T + D)
    got = _run_gpu(x, gx, ga, go, lam, torch.float32)
    _check(got, _oracle(x, gx, ga, go, lam, got[0]), FP32_TOL)


@pytest.mark.parametrize("B,T,D", SHAPES)
def test_scan_bf16_matches_oracle(B, T, D):
    x, gx, ga, go, lam = _inputs(B, T, D, seed=7 + B * 1000 + T + D, dtype=torch.bfloat16)
    got = _run_gpu(x, gx, ga, go, lam, torch.bfloat16)
    _check(got, _oracle(x, gx, ga, go, lam, got[0]), BF16_TOL)


def test_scan_config0_fp32():
    """B=2, T=2048, D=512, fp32, h0=0, Lambda on the 0.9..0.999 ring, seed 0."""
    torch.manual_seed(0)
    x, gx, ga, go = (torch.randn(2, 2048, 512) for _ in range(4))
    lam = oscan.rnn_param_ring(512)
    got = _run_gpu(x, gx, ga, go, lam, torch.float32)
    want = _oracle(x, gx, ga, go, lam, got[0])
    _check(got, want, FP32_TOL)
    assert max_rel(got[0][:, -1], want[0][:, -1]) <= FP32_TOL  # final state h_T = h[:, -1]


def test_scan_extreme_gates_hit_sqrt_grad_clamp():
    """Gate pre-activations of +-20 saturate a -> 1, where the reference clamps d sqrt (scan_fused.py:10-15)."""
    x, gx, ga, go, lam = _inputs(2, 96, 64, seed=11, scale=8.0)
    ga[:, ::3] = -20.0
    gx[:, 1::3] = 20.0
    got = _run_gpu(x, gx, ga, go, lam, torch.float32)
    assert all(torch.isfinite(t).all() for t in got)
    # 1 - a^2 cancels catastrophically in fp32 when a -> 1; the fp32 oracle has the same arithmetic
    h32 = oscan.rglru_scan_fwd(x, gx, ga, lam)
    g32 = oscan.rglru_scan_bwd(x, gx, ga, lam, got[0], go)
    _check(got, (h32,) + g32, 1e-3)


@pytest.mark.parametrize("lo,hi", [(-9.0, -4.0), (-6.0, -2.0), (3.0, 8.0)])
def test_scan_bf16_saturated_recurrence_gate(lo, hi):
    """Recurrence gates deep in saturation over a long sequence: with r <= 0.02 the decay a = exp(-8 r softplus)
    sits within 1e-3 of 1 and small errors of r accumulate over ~1/(1-a) steps (the bf16 kernels evaluate the
    sigmoids with one approximate transcendental each); with r -> 1 the state forgets fastest.  Forward and
    every gradient stay inside the bf16 bound against the fp64 oracle."""
    B, T, D = 2, 4096, 128
    g = torch.Generator().manual_seed(int(100 - lo))
    x, gx, go = (torch.randn(B, T, D, generator=g) for _ in range(3))
    ga = lo + (hi - lo) * torch.rand(B, T, D, generator=g)
    lam = oscan.rnn_param_ring(D, generator=g)
    x, gx, ga, go = (t.to(torch.bfloat16).float() for t in (x, gx, ga, go))
    got = _run_gpu(x, gx, ga, go, lam, torch.bfloat16)
    _check(got, _oracle(x, gx, ga, go, lam, got[0]), BF16_TOL)


def test_scan_closed_form_known_answer():
    lam = oscan.rnn_param_ring(64, generator=torch.Generator().manual_seed(3))
    T = 700
    ones, zeros = torch.ones(1, T, 64), torch.zeros(1, T, 64)
    got = _run_gpu(ones, zeros, zeros, zeros, lam, torch.float32)
    assert max_rel(got[0], oscan.closed_form_kat(lam, T)) <= FP32_TOL


def test_scan_matches_reference_triton_golden():
    """Against outputs of the reference's own kernels (bf16-truncating stores): within bf16 rounding."""
    g = load_golden("scan_triton_interp.npz")
    for tag in "abc":
        x, gx, ga, go, lam = (g[f"{tag}_{k}"] for k in ("x", "gx", "ga", "go", "lam"))
        if x.shape[1] < 2:
            continue
        got = _run_gpu(x, gx, ga, go, lam, torch.float32)
        for n, a in zip(("h", "dx", "dgx", "dga", "dlam"), got):
            assert max_rel(a, g[f"{tag}_{n}"]) <= 2e-2, (tag, n)


def test_scan_autocast_casts_like_the_reference():
    from hawk_b200 import fused_linear_scan
    x, gx, ga, go, lam = _inputs(2, 40, 64, seed=5)
    xs = [t.cuda().requires_grad_(True) for t in (x, gx, ga)]
    with torch.autocast("cuda", dtype=torch.bfloat16):
        h = fused_linear_scan(*xs, lam.cuda())
    assert h.dtype == torch.bfloat16
    h.float().sum().backward()
    assert all(t.grad.dtype == torch.float32 for t in xs)
    want = oscan.rglru_scan_fwd(*(t.bfloat16().float() for t in (x, gx, ga)), lam, compute=torch.float64)
    assert rel_l2(h.float().cpu(), want) <= BF16_TOL


def test_scan_noncontiguous_inputs_and_initial_state():
    x, gx, ga, go, lam = _inputs(2, 70, 128, seed=9)
    h0 = torch.randn(2, 128, generator=torch.Generator().manual_seed(1))
    big = torch.randn(2, 70, 256)
    big[..., :128] = x
    from hawk_b200 import fused_linear_scan
    hv = fused_linear_scan(big.cuda()[..., :128], gx.cuda(), ga.cuda(), lam.cuda())
    assert rel_l2(hv.cpu(), oscan.rglru_scan_fwd(x, gx, ga, lam, compute=torch.float64)) <= FP32_TOL
    got = _run_gpu(x, gx, ga, go, lam, torch.float32, h0=h0)
    ref = oscan.rglru_scan_autograd  # differentiable fp64 statement, extended with h0 below
    xs = [t.double().requires_grad_(True) for t in (x, gx, ga, lam, h0)]
    sp = torch.nn.functional.softplus(xs[3])
    a = torch.exp(-8.0 * torch.sigmoid(xs[2]) * sp)
    beta = xs[0] * torch.sigmoid(xs[1]) * torch.sqrt(1 - a * a)
    hs, st = [], xs[4]
    for t in range(x.shape[1]):
        st = a[:, t] * st + beta[:, t]
        hs.append(st)
    h = torch.stack(hs, 1)
    grads = torch.autograd.grad(h, xs, go.double())
    _check(got, (h.detach(),) + grads, FP32_TOL, names=("h", "dx", "dgx", "dga", "dlam", "dh0"))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, BF16_TOL)])
@pytest.mark.parametrize("B,T,D", [(1, 1, 64), (2, 33, 64), (3, 257, 192), (2, 2048, 512), (8, 300, 2048)])
def test_scan_gate_bias_equals_bias_added_outside(B, T, D, dtype, tol):
    """gate_bias=[bx; ba] inside the kernel == the oracle run on (gx + bx, ga + ba), which is what the
    reference's block-diagonal projections hand its scan (hawk/hawk.py:128-129); the bias gradients
    are the sums of d gx, d ga over batch and time (autograd of the broadcast add)."""
    from hawk_b200 import fused_linear_scan
    x, gx, ga, go, lam = _inputs(B, T, D, seed=31 + B + T + D, dtype=dtype)
    g = torch.Generator().manual_seed(5)
    gb = torch.randn(2, D, generator=g)
    gb[0, ::7] = -40.0   # far below the kernel's internal floor: the gate is 0 either way
    gb[1, 3::11] = 25.0  # saturated recurrence gate
    dev = "cuda:0"
    xs = [t.to(dev, dtype).requires_grad_(True) for t in (x, gx, ga)]
    lam_d = lam.to(dev).requires_grad_(True)
    gb_d = gb.to(dev).requires_grad_(True)
    h = fused_linear_scan(*xs, lam_d, gate_bias=gb_d)
    h.backward(go.to(dev, dtype))
    got = [t.float().cpu() for t in (h.detach(), xs[0].grad, xs[1].grad, xs[2].grad, lam_d.grad, gb_d.grad)]
    gxb, gab = gx + gb[0], ga + gb[1]
    wh, wdx, wdgx, wdga, wdlam = _oracle(x, gxb, gab, go, lam, got[0])
    want = (wh, wdx, wdgx, wdga, wdlam, torch.stack((wdgx.sum((0, 1)), wdga.sum((0, 1)))))
    _check(got, want, tol, names=("h", "dx", "dgx", "dga", "dlam", "dgate_bias"))
    # the bias gradient is the fixed-order sum of the gate gradients the kernel itself stored
    if dtype == torch.float32:
        own = torch.stack((got[2].double().sum((0, 1)), got[3].double().sum((0, 1)))).float()
        assert rel_l2(got[5], own) <= 1e-5


def test_scan_is_deterministic():
    x, gx, ga, go, lam = _inputs(4, 300, 256, seed=21, dtype=torch.bfloat16)
    a = _run_gpu(x, gx, ga, go, lam, torch.bfloat16)
    b = _run_gpu(x, gx, ga, go, lam, torch.bfloat16)
    assert all(torch.equal(p, q) for p, q in zip(a, b))


def test_scan_metric_shape_properties():
    """B=8, T=4096, D=2048 bf16 (too large for the CPU oracle in seconds): size-independent checks.
    (1) time-locality: h[:, :t] does not depend on inputs after t; (2) a channel slice scanned alone gives
    the same h up to last-bit bf16 roundings (that launch has few channel groups and is cut in time across
    CTAs, which associates the fp32 recurrence differently); (3) a sampled set of channels matches the fp64
    oracle."""
    from hawk_b200 import fused_linear_scan
    B, T, D = 8, 4096, 2048
    g = torch.Generator(device="cuda").manual_seed(0)
    x, gx, ga, go = (torch.randn(B, T, D, generator=g, device="cuda").bfloat16() for _ in range(4))
    lam = oscan.rnn_param_ring(D, generator=torch.Generator().manual_seed(0)).cuda()
    xs = [t.clone().requires_grad_(True) for t in (x, gx, ga)]
    lam_r = lam.clone().requires_grad_(True)
    h = fused_linear_scan(*xs, lam_r)
    h.backward(go)
    # (1)
    h_half = fused_linear_scan(x[:, :1000].contiguous(), gx[:, :1000].contiguous(), ga[:, :1000].contiguous(), lam)
    assert torch.equal(h_half, h[:, :1000])
    # (2)
    sl = slice(640, 704)
    h_sl = fused_linear_scan(x[..., sl].contiguous(), gx[..., sl].contiguous(), ga[..., sl].contiguous(), lam[sl].contiguous())
    assert rel_l2(h_sl.float(), h[..., sl].detach().float()) <= 2e-3
    # (3)
    idx = torch.tensor([0, 1, 63, 64, 777, 1024, 2046, 2047])
    cx, cgx, cga, cgo = (t[:2][..., idx.cuda()].float().cpu() for t in (x, gx, ga, go))
    hs = h.detach()[:2][..., idx.cuda()].float().cpu()
    want_h = oscan.rglru_scan_fwd(cx, cgx, cga, lam.cpu()[idx], compute=torch.float64)
    assert rel_l2(hs, want_h) <= BF16_TOL
    wdx, wdgx, wdga, _ = oscan.rglru_scan_bwd(cx, cgx, cga, lam.cpu()[idx], hs.double(), cgo, compute=torch.float64)
    for a, b in zip((xs[0].grad, xs[1].grad, xs[2].grad), (wdx, wdgx, wdga)):
        assert rel_l2(a[:2][..., idx.cuda()].float().cpu(), b) <= BF16_TOL
    assert torch.isfinite(lam_r.grad).all()


def test_scan_long_sequence_shape_properties():
    """B=1, T=65536, D=4096 bf16 (the long-sequence stress shape; 268 M elements): (1) time-locality over a
    prefix that ends inside a super-step; (2) a 64-channel slice scanned alone (a launch small enough to be cut
    in time across CTAs) gives the same h up to last-bit bf16 roundings; (3) sampled channels match the fp64 oracle over all 65536 steps, forward and backward, with
    gate biases inside the kernel."""
    from hawk_b200 import fused_linear_scan
    B, T, D = 1, 65536, 4096
    g = torch.Generator(device="cuda").manual_seed(4)
    x, gx, ga, go = (torch.randn(B, T, D, generator=g, device="cuda").bfloat16() for _ in range(4))
    lam = oscan.rnn_param_ring(D, generator=torch.Generator().manual_seed(4)).cuda()
    gb = 0.3 * torch.randn(2, D, generator=g, device="cuda")
    xs = [t.clone().requires_grad_(True) for t in (x, gx, ga)]
    lam_r, gb_r = lam.clone().requires_grad_(True), gb.clone().requires_grad_(True)
    h = fused_linear_scan(*xs, lam_r, gate_bias=gb_r)
    h.backward(go)
    assert bool(torch.isfinite(h).all())
    # (1)
    tcut = 40001
    h_pre = fused_linear_scan(x[:, :tcut].contiguous(), gx[:, :tcut].contiguous(), ga[:, :tcut].contiguous(), lam,
                              gate_bias=gb)
    assert torch.equal(h_pre, h.detach()[:, :tcut])
    # (2)
    sl = slice(2048, 2112)
    h_sl = fused_linear_scan(x[..., sl].contiguous(), gx[..., sl].contiguous(), ga[..., sl].contiguous(),
                             lam[sl].contiguous(), gate_bias=gb[:, sl].contiguous())
    assert rel_l2(h_sl.float(), h.detach()[..., sl].float()) <= 2e-3
    # (3)
    idx = torch.tensor([0, 65, 2047, 4095])
    ic = idx.cuda()
    cx, cgx, cga, cgo = (t[..., ic].float().cpu() for t in (x, gx, ga, go))
    cgb = gb[:, ic].cpu()
    cgx, cga = cgx + cgb[0], cga + cgb[1]
    hs = h.detach()[..., ic].float().cpu()
    lam_c = lam.cpu()[idx]
    want_h = oscan.rglru_scan_fwd(cx, cgx, cga, lam_c, compute=torch.float64)
    assert rel_l2(hs, want_h) <= BF16_TOL
    wdx, wdgx, wdga, wdlam = oscan.rglru_scan_bwd(cx, cgx, cga, lam_c, hs.double(), cgo, compute=torch.float64)
    for a, b in zip((xs[0].grad, xs[1].grad, xs[2].grad), (wdx, wdgx, wdga)):
        assert rel_l2(a[..., ic].float().cpu(), b) <= BF16_TOL
    assert rel_l2(lam_r.grad[ic].cpu(), wdlam) <= BF16_TOL
    want_gb = torch.stack((wdgx.sum((0, 1)), wdga.sum((0, 1))))
    assert rel_l2(gb_r.grad[:, ic].cpu(), want_gb) <= BF16_TOL


def test_reference_host_function_names():
    """sequential_scan_forward / sequential_scan_backward with the reference's argument order
    (hawk/scan_fused.py:319-324,363-370) give what fused_linear_scan and its autograd give."""
    from hawk_b200 import fused_linear_scan, sequential_scan_backward, sequential_scan_forward
    x, gx, ga, go, lam = _inputs(2, 130, 128, seed=21)
    xs = [t.cuda().requires_grad_(True) for t in (x, gx, ga)]
    lam_d = lam.cuda().requires_grad_(True)
    h = fused_linear_scan(*xs, lam_d)
    h.backward(go.cuda())
    h2 = sequential_scan_forward(x.cuda(), gx.cuda(), ga.cuda(), lam.cuda())
    assert torch.equal(h2, h.detach())
    grads = sequential_scan_backward(x.cuda(), gx.cuda(), ga.cuda(), lam.cuda(), h2, go.cuda())
    for a, b in zip(grads, (xs[0].grad, xs[1].grad, xs[2].grad, lam_d.grad)):
        assert torch.equal(a, b)
