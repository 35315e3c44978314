"""The scan with the block's epilogue fused in (out = gelu(y) * h, hawk/hawk.py:134-135,186,201), through
the C ABI, against the CPU oracle: oracle scan (fp64) followed by torch's exact GELU in fp64, gradients of
the epilogue from autograd and of the scan from the restated reference backward.

Tolerances as for the plain scan: fp32 storage <= 1e-5, bf16 storage <= 2e-2, norm-wise.
"""
import pytest
import torch
import torch.nn.functional as F

from conftest import max_rel, rel_l2
from oracle import scan as oscan

pytestmark = pytest.mark.gpu


def _inputs(B, T, D, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    x, gx, ga, dout = (torch.randn(B, T, D, generator=g) for _ in range(4))
    xy = torch.randn(B, T, 2 * D, generator=g) * 1.5  # y is the strided second half, as in the block
    gb = 0.3 * torch.randn(2, D, generator=g)
    lam = oscan.rnn_param_ring(D, generator=g)
    if dtype != torch.float32:
        x, gx, ga, dout, xy = (t.to(dtype).float() for t in (x, gx, ga, dout, xy))
    return x, gx, ga, dout, xy, gb, lam


def _oracle(x, gx, ga, dout, y, gb, lam, h_stored):
    gxb, gab = (gx + gb[0]).double(), (ga + gb[1]).double()
    h = oscan.rglru_scan_fwd(x, gxb, gab, lam, compute=torch.float64)
    yd = y.double().requires_grad_(True)
    gelu = F.gelu(yd)
    out = gelu * h
    dgelu, = torch.autograd.grad(gelu.sum(), yd)
    dh = dout.double() * gelu.detach()
    dx, dgx, dga, dlam = oscan.rglru_scan_bwd(x, gxb, gab, lam, h_stored.double(), dh, compute=torch.float64)
    dy = dout.double() * h * dgelu
    return dict(h=h, out=out.detach(), dx=dx, dgx=dgx, dga=dga, dlam=dlam, dy=dy,
                dgb=torch.stack((dgx.sum((0, 1)), dga.sum((0, 1)))))


def _run(x, gx, ga, dout, xy, gb, lam, dtype, use_bias):
    from hawk_b200 import fused_scan_gelu
    dev = "cuda:0"
    D = x.shape[-1]
    xs = [t.to(dev, dtype).requires_grad_(True) for t in (x, gx, ga)]
    xyd = xy.to(dev, dtype).requires_grad_(True)
    lam_d = lam.to(dev).requires_grad_(True)
    gb_d = gb.to(dev).requires_grad_(True) if use_bias else None
    out, h = fused_scan_gelu(*xs, lam_d, xyd[..., D:], gate_bias=gb_d)
    assert out.dtype == dtype and h.dtype == dtype and not h.requires_grad
    out.backward(dout.to(dev, dtype))
    assert float(xyd.grad[..., :D].abs().max()) == 0.0  # the x half of the projection is not an input here
    res = dict(h=h.detach(), out=out.detach(), dx=xs[0].grad, dgx=xs[1].grad, dga=xs[2].grad, dlam=lam_d.grad,
               dy=xyd.grad[..., D:])
    if use_bias:
        res["dgb"] = gb_d.grad
    return {k: v.float().cpu() for k, v in res.items()}


SHAPES = [(1, 1, 64), (2, 3, 128), (2, 33, 64), (1, 65, 128), (3, 257, 192), (2, 2048, 512), (1, 1000, 4096),
          (8, 300, 2048)]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("B,T,D", SHAPES)
def test_fused_scan_gelu_matches_oracle(B, T, D, dtype, tol):
    x, gx, ga, dout, xy, gb, lam = _inputs(B, T, D, seed=B * 1000 + T + D, dtype=dtype)
    use_bias = (B + T) % 2 == 0
    got = _run(x, gx, ga, dout, xy, gb, lam, dtype, use_bias)
    zero = torch.zeros_like(gb)
    want = _oracle(x, gx, ga, dout, xy[..., D:], gb if use_bias else zero, lam, got["h"])
    for k, v in got.items():
        assert rel_l2(v, want[k]) <= tol, (k, rel_l2(v, want[k]))
        assert max_rel(v, want[k]) <= tol, (k, max_rel(v, want[k]))


def test_fused_equals_separate_kernels_bf16():
    """Same tensors through the fused kernels and through scan + gelu_mul: h, out and the gradients within bf16
    rounding of each other (the two paths use different launch shapes, so the fp32 recurrence is associated
    differently and h may differ in the last bf16 bit)."""
    from hawk_b200 import fused_linear_scan, fused_scan_gelu, ops
    B, T, D = 8, 1024, 2048
    x, gx, ga, dout, xy, gb, lam = _inputs(B, T, D, seed=5, dtype=torch.bfloat16)
    dev, dt = "cuda:0", torch.bfloat16

    def leaves():
        return ([t.to(dev, dt).requires_grad_(True) for t in (x, gx, ga)], xy.to(dev, dt).requires_grad_(True),
                lam.to(dev).requires_grad_(True), gb.to(dev).requires_grad_(True))
    xs, xyd, lam_d, gb_d = leaves()
    out, h = fused_scan_gelu(*xs, lam_d, xyd[..., D:], gate_bias=gb_d)
    out.backward(dout.to(dev, dt))
    xs2, xyd2, lam2, gb2 = leaves()
    h2 = fused_linear_scan(*xs2, lam2, gate_bias=gb2)
    out2 = ops.gelu_mul(xyd2[..., D:], h2)
    out2.backward(dout.to(dev, dt))
    assert rel_l2(h.float(), h2.float()) <= 2e-3
    assert rel_l2(out.float(), out2.float()) <= 4e-3
    for a, b in zip(xs + [xyd, lam_d, gb_d], xs2 + [xyd2, lam2, gb2]):
        assert rel_l2(a.grad.float(), b.grad.float()) <= 8e-3


def test_fused_scan_gelu_metric_shape_properties():
    """B=8, T=4096, D=2048 bf16 (the benchmark's scan shape): time locality (a prefix of the sequence gives
    the same prefix of h and out, bit for bit) and sampled channels against the fp64 oracle."""
    from hawk_b200 import fused_scan_gelu
    B, T, D = 8, 4096, 2048
    g = torch.Generator(device="cuda").manual_seed(3)
    x, gx, ga = (torch.randn(B, T, D, generator=g, device="cuda").bfloat16() for _ in range(3))
    xy = torch.randn(B, T, 2 * D, generator=g, device="cuda").bfloat16()
    lam = oscan.rnn_param_ring(D, generator=torch.Generator().manual_seed(4)).cuda()
    out, h = fused_scan_gelu(x, gx, ga, lam, xy[..., D:])
    out_p, h_p = fused_scan_gelu(x[:, :1000].contiguous(), gx[:, :1000].contiguous(), ga[:, :1000].contiguous(), lam,
                                 xy[:, :1000, D:])
    assert torch.equal(h[:, :1000], h_p) and torch.equal(out[:, :1000], out_p)
    ch = torch.arange(0, D, 97)
    hw = oscan.rglru_scan_fwd(x[..., ch].float().cpu(), gx[..., ch].float().cpu(), ga[..., ch].float().cpu(),
                              lam[ch].cpu(), compute=torch.float64)
    want = F.gelu(xy[..., D:][..., ch].double().cpu()) * hw
    assert rel_l2(out[..., ch].float().cpu(), want) <= 2e-2
