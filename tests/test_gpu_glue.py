"""The fused glue kernels (gelu(a)*b, RMSNorm, block-diagonal gate pair) against plain PyTorch fp32
statements of the same ops.  fp32 <= 1e-5, bf16 <= 2e-2, norm-wise."""
import pytest
import torch
import torch.nn.functional as F

from conftest import max_rel, rel_l2
from oracle import model as omodel

pytestmark = pytest.mark.gpu


def _tol(dtype):
    return 1e-5 if dtype == torch.float32 else 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,J", [(1, 8), (7, 64), (300, 1024), (4096, 6144)])
def test_geglu_and_strided_gelu_mul(dtype, M, J):
    from hawk_b200 import ops
    g = torch.Generator().manual_seed(M + J)
    gu = (2 * torch.randn(M, 2 * J, generator=g)).to(dtype)
    go = torch.randn(M, J, generator=g).to(dtype)
    ref_in = gu.float().double().requires_grad_(True)
    ref = F.gelu(ref_in[:, :J]) * ref_in[:, J:]
    ref.backward(go.double())
    # fused whole-buffer form
    x = gu.cuda().requires_grad_(True)
    out = ops.geglu(x)
    out.backward(go.cuda())
    assert rel_l2(out.float().cpu(), ref.detach()) <= _tol(dtype)
    assert rel_l2(x.grad.float().cpu(), ref_in.grad) <= _tol(dtype)
    assert max_rel(x.grad.float().cpu(), ref_in.grad) <= _tol(dtype)
    # strided-view form: a is the second half of a buffer, b contiguous (as gelu(y) * h in the block)
    buf = gu.cuda().requires_grad_(True)
    b = go.cuda().clone().requires_grad_(True)
    out2 = ops.gelu_mul(buf[:, J:], b)
    out2.backward(torch.ones_like(out2))
    r_a = gu[:, J:].double().requires_grad_(True)
    r_b = go.double().requires_grad_(True)
    (F.gelu(r_a) * r_b).sum().backward()
    assert rel_l2(out2.float().cpu(), (F.gelu(r_a) * r_b).detach()) <= _tol(dtype)
    assert rel_l2(buf.grad[:, J:].float().cpu(), r_a.grad) <= _tol(dtype)
    assert float(buf.grad[:, :J].abs().max()) == 0.0
    assert rel_l2(b.grad.float().cpu(), r_b.grad) <= _tol(dtype)


def test_bf16_gelu_is_the_erf_gelu_on_every_bf16_value():
    """The bf16 kernels evaluate the exact GELU in logistic form (polynomial logit of the normal CDF);
    on EVERY finite bf16 input the result is the erf GELU to within one bf16 rounding step, forward and
    derivative, including the saturated tails and the largest magnitudes."""
    from hawk_b200 import ops
    bits = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16)
    a = bits.view(torch.bfloat16)
    a = a[torch.isfinite(a)]
    n = a.numel() // 8 * 8
    a = a[:n].reshape(1, n).cuda()
    one = torch.ones_like(a)
    out = ops.gelu_mul_fwd(a, one)
    da, db = ops.gelu_mul_bwd(one, a, one)
    ad = a.double().cpu()
    cdf = 0.5 * torch.erfc(-ad / 2 ** 0.5)
    want = ad * cdf
    dwant = cdf + ad * torch.exp(-0.5 * ad * ad) / (2 * torch.pi) ** 0.5
    for got, ref in ((out, want), (db, want), (da, dwant)):
        err = (got.double().cpu() - ref).abs()
        assert bool((err <= 2.0 ** -7 * ref.abs() + 1e-7).all()), float((err / (ref.abs() + 1e-7)).max())
        assert bool(torch.isfinite(got).all())


@pytest.mark.parametrize("xdt,ydt", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                     (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("M,H", [(1, 64), (33, 512), (2, 1024), (1000, 2048), (257, 4096), (1, 2048), (600, 384)])
def test_rms_norm_matches_torch(xdt, ydt, M, H):
    from hawk_b200 import ops
    g = torch.Generator().manual_seed(M + H)
    x = (3 * torch.randn(M, H, generator=g)).to(xdt)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    go = torch.randn(M, H, generator=g).to(ydt)
    xr = x.double().requires_grad_(True)
    wr = w.double().requires_grad_(True)
    ref = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    ref.backward(go.double())
    xd = x.cuda().requires_grad_(True)
    wd = w.cuda().requires_grad_(True)
    y = ops.rms_norm(xd, wd, 1e-6, out_dtype=ydt)
    assert y.dtype == ydt
    y.backward(go.cuda())
    assert rel_l2(y.float().cpu(), ref.detach()) <= _tol(ydt)
    assert rel_l2(xd.grad.float().cpu(), xr.grad) <= _tol(xdt if xdt == ydt else ydt)
    assert rel_l2(wd.grad.cpu(), wr.grad) <= (1e-5 if ydt == torch.float32 else 2e-2)
    # determinism of the two-stage weight-gradient reduction
    xd2 = x.cuda().requires_grad_(True)
    wd2 = w.cuda().requires_grad_(True)
    ops.rms_norm(xd2, wd2, 1e-6, out_dtype=ydt).backward(go.cuda())
    assert torch.equal(wd.grad, wd2.grad) and torch.equal(xd.grad, xd2.grad)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nb,bw,lead", [(4, 16, (2, 5)), (16, 32, (3, 100)), (16, 128, (2, 300))])
def test_block_diag_gates_match_einsum(dtype, nb, bw, lead):
    from hawk_b200 import ops
    g = torch.Generator().manual_seed(nb + bw)
    R = nb * bw
    x = torch.randn(*lead, R, generator=g).to(dtype)
    ws = [torch.randn(nb, bw, bw, generator=g) / bw ** 0.5 for _ in range(2)]
    bs = [0.1 * torch.randn(nb, bw, generator=g) for _ in range(2)]
    gos = [torch.randn(*lead, R, generator=g).to(dtype) for _ in range(2)]
    xr = x.double().requires_grad_(True)
    pr = [t.double().requires_grad_(True) for t in (ws[0], bs[0], ws[1], bs[1])]
    r1 = omodel.block_diag_linear(xr, pr[0], pr[1])
    r2 = omodel.block_diag_linear(xr, pr[2], pr[3])
    torch.autograd.backward([r1, r2], [gos[0].double(), gos[1].double()])
    xd = x.cuda().requires_grad_(True)
    pd = [t.cuda().requires_grad_(True) for t in (ws[0], bs[0], ws[1], bs[1])]
    o1, o2 = ops.block_diag_gates(xd, *pd)
    assert o1.is_contiguous() and o2.is_contiguous() and o1.dtype == dtype
    torch.autograd.backward([o1, o2], [gos[0].cuda(), gos[1].cuda()])
    tol = _tol(dtype) if dtype == torch.bfloat16 else 2e-3  # fp32 bmm may run as TF32 on tensor cores
    assert rel_l2(o1.float().cpu(), r1.detach()) <= tol and rel_l2(o2.float().cpu(), r2.detach()) <= tol
    assert rel_l2(xd.grad.float().cpu(), xr.grad) <= tol
    for a, b in zip(pd, pr):
        assert rel_l2(a.grad.cpu(), b.grad) <= tol


@pytest.mark.parametrize("xdt,ydt", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                     (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("M,H", [(5, 64), (300, 2048), (1, 512), (700, 1024), (77, 4096), (593, 2048)])
def test_add_rms_norm_matches_torch(xdt, ydt, M, H):
    """Fused residual add + norm: both outputs and all three gradients, with gradient arriving on the
    summed residual as well as on the norm output."""
    from hawk_b200 import ops
    g = torch.Generator().manual_seed(M * 7 + H)
    res = (2 * torch.randn(M, H, generator=g)).to(xdt)
    delta = torch.randn(M, H, generator=g).to(ydt)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    g_y = torch.randn(M, H, generator=g).to(ydt)
    g_r = torch.randn(M, H, generator=g).to(xdt)
    rr, dr, wr = res.double().requires_grad_(True), delta.double().requires_grad_(True), w.double().requires_grad_(True)
    s = rr + dr
    if xdt == torch.bfloat16:
        s = s + (s.detach().bfloat16().double() - s.detach())  # the stream is stored in bf16
    yr = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    torch.autograd.backward([s, yr], [g_r.double(), g_y.double()])
    rd, dd, wd = res.cuda().requires_grad_(True), delta.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    new_res, y = ops.add_rms_norm(rd, dd, wd, 1e-6, out_dtype=ydt)
    assert new_res.dtype == xdt and y.dtype == ydt
    torch.autograd.backward([new_res, y], [g_r.cuda(), g_y.cuda()])
    tol = 1e-5 if (xdt == torch.float32 and ydt == torch.float32) else 2e-2
    assert rel_l2(new_res.float().cpu(), s.detach()) <= (1e-6 if xdt == torch.float32 else 1e-2)
    assert rel_l2(y.float().cpu(), yr.detach()) <= tol
    assert rel_l2(rd.grad.float().cpu(), rr.grad) <= tol
    assert rel_l2(dd.grad.float().cpu(), dr.grad) <= tol
    assert rel_l2(wd.grad.cpu(), wr.grad) <= tol
    # residual-only gradient (norm output unused) and norm-only gradient (sum unused)
    rd2, dd2 = res.cuda().requires_grad_(True), delta.cuda().requires_grad_(True)
    nr2, y2 = ops.add_rms_norm(rd2, dd2, wd.detach(), 1e-6, out_dtype=ydt)
    nr2.backward(g_r.cuda())
    assert rel_l2(rd2.grad.float().cpu(), g_r.double()) <= 1e-6
    rd3, dd3 = res.cuda().requires_grad_(True), delta.cuda().requires_grad_(True)
    _, y3 = ops.add_rms_norm(rd3, dd3, wd.detach(), 1e-6, out_dtype=ydt)
    y3.backward(g_y.cuda())
    assert torch.isfinite(rd3.grad).all() and rel_l2(dd3.grad.float().cpu(), rd3.grad.float().cpu()) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,T,R,nb", [(2, 33, 64, 2), (3, 200, 256, 4), (1, 1, 128, 16)])
def test_recurrent_core_equals_the_separate_operators(dtype, B, T, R, nb):
    """One autograd node for conv -> gates -> scan -> gelu(y) * h: same outputs and the same gradients as
    the chain of separate operators (chunk, Conv1D, block-diagonal gates with biases, scan, gelu_mul)."""
    from hawk_b200 import ops
    g = torch.Generator().manual_seed(B * 100 + T + R)
    bw = R // nb
    xy = torch.randn(B, T, 2 * R, generator=g).to(dtype)
    cw, cb = 0.3 * torch.randn(4, R, generator=g), 0.1 * torch.randn(R, generator=g)
    wx, wa = (torch.randn(nb, bw, bw, generator=g) / bw ** 0.5 for _ in range(2))
    bx, ba = (0.2 * torch.randn(nb, bw, generator=g) for _ in range(2))
    lam = torch.rand(R, generator=g) * 4 - 6
    go = torch.randn(B, T, R, generator=g).to(dtype)

    def leaves():
        return [t.clone().cuda().requires_grad_(True) for t in (xy, cw, cb, wx, wa, bx, ba, lam)]

    a = leaves()
    out, h = ops.recurrent_core(a[0], a[1], a[2], a[3], a[4], torch.stack((a[5].reshape(-1), a[6].reshape(-1))), a[7])
    assert not h.requires_grad
    out.backward(go.cuda())
    b = leaves()
    xb, y = b[0].chunk(2, dim=-1)
    xc = ops.temporal_conv1d(xb, b[1], b[2], out_dtype=dtype)
    gx, ga = ops.block_diag_gates(xc, b[3], b[5], b[4], b[6])
    h2 = ops.fused_linear_scan(xc, gx, ga, b[7])
    out2 = ops.gelu_mul(y, h2)
    out2.backward(go.cuda())
    tol = 2e-3 if dtype == torch.float32 else 3e-2  # fp32 bmm may run as TF32; bf16 rounds gate + bias once more
    assert rel_l2(out.float().cpu(), out2.float().cpu()) <= tol and rel_l2(h.float().cpu(), h2.float().cpu()) <= tol
    for name, p, q in zip(("xy", "conv_w", "conv_b", "wx", "wa", "bx", "ba", "lam"), a, b):
        assert p.grad is not None and p.grad.shape == q.grad.shape, name
        assert rel_l2(p.grad.float().cpu(), q.grad.float().cpu()) <= tol, (name, rel_l2(p.grad.float().cpu(), q.grad.float().cpu()))


@pytest.mark.parametrize("n", [1, 7, 8, 9, 4099, 1 << 20, (1 << 22) + 3])
def test_cast_bf16_is_bit_exact_round_to_nearest_even(n):
    from hawk_b200 import ops
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=g) * torch.exp(8 * torch.randn(n, generator=g))
    special = torch.tensor([0.0, -0.0, float("inf"), -float("inf"), 1.00390625, 1.01171875, 3.3e38, -3.4e38, 1e-40,
                            float("nan")])
    x[:min(n, special.numel())] = special[:min(n, special.numel())]
    got = ops.cast_bf16(x.cuda())
    want = x.cuda().to(torch.bfloat16)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("lead,K,N", [((3, 50), 64, 96), ((1000,), 512, 256), ((2, 7, 9), 128, 40)])
def test_autocast_linear_matches_f_linear(lead, K, N):
    """ops.linear under bf16 autocast: the same output and input gradient as F.linear (bit for bit: same
    rounded operands, same GEMM), the weight gradient in fp32 straight from the GEMM (at least as close to
    the exact product as autocast's bf16-rounded one); outside autocast it is F.linear."""
    from hawk_b200 import ops
    g = torch.Generator().manual_seed(K + N)
    x = torch.randn(*lead, K, generator=g)
    w = torch.randn(N, K, generator=g) / K ** 0.5
    go = torch.randn(*lead, N, generator=g)
    outs = []
    for fn in (ops.linear, F.linear):
        xd, wd = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = fn(xd, wd)
        assert y.dtype == torch.bfloat16
        y.backward(go.cuda().to(y.dtype))
        assert xd.grad.dtype == torch.float32 and wd.grad.dtype == torch.float32
        outs.append((y.detach(), xd.grad, wd.grad))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    xb, gb = x.bfloat16().double().reshape(-1, K), go.bfloat16().double().reshape(-1, N)
    exact = gb.t() @ xb
    e_mine, e_auto = rel_l2(outs[0][2].cpu(), exact), rel_l2(outs[1][2].cpu(), exact)
    assert e_mine <= 1e-5 and e_mine <= e_auto + 1e-7, (e_mine, e_auto)
    xd, wd = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    y = ops.linear(xd, wd)  # no autocast: plain fp32 F.linear
    assert y.dtype == torch.float32 and rel_l2(y.detach().cpu(), F.linear(x, w)) <= 2e-3
