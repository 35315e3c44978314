"""Parity of the CUDA conv1d and decode-step kernels (through the C ABI) with the CPU oracle and
with the fixtures produced by the reference modules.  fp32: <= 1e-5 norm-wise; bf16: <= 2e-2."""
import pytest
import torch

from conftest import load_golden, max_rel, rel_l2
from oracle import conv1d as oconv
from oracle import decode as odec
from oracle import scan as oscan

pytestmark = pytest.mark.gpu
FP32_TOL = 1e-5
BF16_TOL = 2e-2


def _conv_gpu(x, w, b, go, dtype, out_dtype=None, strided=True):
    from hawk_b200 import temporal_conv1d
    B, T, D = x.shape
    if strided:  # the x half of a [B,T,2D] projection, as torch.chunk gives in the model
        xy = torch.zeros(B, T, 2 * D, dtype=dtype, device="cuda")
        xy[..., :D] = x.to("cuda", dtype)
        xy.requires_grad_(True)
        xv = xy[..., :D]
    else:
        xy = x.to("cuda", dtype).requires_grad_(True)
        xv = xy
    wd, bd = w.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    y = temporal_conv1d(xv, wd, bd, out_dtype=out_dtype)
    y.backward(go.to("cuda", y.dtype))
    dx = xy.grad[..., :D] if strided else xy.grad
    return y.detach().float().cpu(), dx.float().cpu(), wd.grad.cpu(), bd.grad.cpu(), y.dtype


def test_conv_matches_reference_fixture():
    g = load_golden("conv1d_ref.npz")
    y, dx, dw, db, ydt = _conv_gpu(g["x"], g["w"], g["b"], g["go"], torch.float32)
    assert ydt == torch.float32
    for a, b in ((y, g["y"]), (dx, g["dx"]), (dw, g["dw"]), (db, g["db"])):
        assert max_rel(a, b) <= FP32_TOL
    from hawk_b200 import temporal_conv1d
    ys = temporal_conv1d(g["short_x"].cuda(), g["w"].cuda(), g["b"].cuda())
    assert max_rel(ys.cpu(), g["short_y"]) <= FP32_TOL


@pytest.mark.parametrize("B,T,D,W", [(1, 1, 8, 4), (2, 3, 64, 4), (2, 31, 72, 4), (3, 100, 512, 4), (1, 257, 1024, 4),
                                     (2, 65, 64, 1), (2, 65, 64, 2), (2, 65, 64, 3), (2, 1024, 2048, 4)])
@pytest.mark.parametrize("strided", [True, False])
def test_conv_fp32_matches_oracle(B, T, D, W, strided):
    g = torch.Generator().manual_seed(B + T + D + W)
    x, go = torch.randn(B, T, D, generator=g), torch.randn(B, T, D, generator=g)
    w, b = torch.randn(W, D, generator=g), torch.randn(D, generator=g)
    y, dx, dw, db, _ = _conv_gpu(x, w, b, go, torch.float32, strided=strided)
    wy = oconv.conv1d_fwd(x, w, b, compute=torch.float64)
    wdx, wdw, wdb = oconv.conv1d_bwd(x, w, go, compute=torch.float64)
    for n, a, bb in (("y", y, wy), ("dx", dx, wdx), ("dw", dw, wdw), ("db", db, wdb)):
        assert rel_l2(a, bb) <= FP32_TOL and max_rel(a, bb) <= FP32_TOL, n


@pytest.mark.parametrize("out_dtype", [None, torch.bfloat16])
def test_conv_bf16_matches_oracle(out_dtype):
    g = torch.Generator().manual_seed(3)
    B, T, D = 2, 300, 256
    x = torch.randn(B, T, D, generator=g).bfloat16().float()
    go = torch.randn(B, T, D, generator=g).bfloat16().float()
    w, b = 0.5 * torch.randn(4, D, generator=g), torch.randn(D, generator=g)
    y, dx, dw, db, ydt = _conv_gpu(x, w, b, go, torch.bfloat16, out_dtype=out_dtype)
    assert ydt == (torch.float32 if out_dtype is None else out_dtype)  # reference promotion: bf16 * fp32 -> fp32
    wy = oconv.conv1d_fwd(x, w, b, compute=torch.float64)
    wdx, wdw, wdb = oconv.conv1d_bwd(x, w, go, compute=torch.float64)
    tol_y = FP32_TOL if out_dtype is None else BF16_TOL
    assert rel_l2(y, wy) <= tol_y
    assert rel_l2(dx, wdx) <= BF16_TOL  # dx is stored in x's dtype (bf16)
    assert rel_l2(dw, wdw) <= FP32_TOL * 10 and rel_l2(db, wdb) <= FP32_TOL * 10


@pytest.mark.parametrize("B,T,D,W", [(1, 1, 64, 4), (2, 3, 64, 4), (1, 15, 128, 4), (2, 16, 64, 4), (1, 17, 192, 4),
                                     (3, 65, 64, 1), (3, 65, 64, 2), (2, 65, 128, 3), (2, 300, 256, 4), (1, 1000, 512, 4),
                                     (2, 4101, 64, 4), (8, 1024, 2048, 4), (1, 4096, 2048, 4)])
@pytest.mark.parametrize("strided", [True, False])
def test_conv_bf16_staged_kernels_match_oracle(B, T, D, W, strided):
    """bf16 in, bf16 out, D a multiple of 64: the shared-memory-staged forward and backward kernels, over
    ragged sequence lengths (shorter than a ring stage, one row past a stage or a tile), every tap count
    (hawk/external.py:49-95) and both input layouts."""
    g = torch.Generator().manual_seed(B + T + D + W)
    x = torch.randn(B, T, D, generator=g).bfloat16().float()
    go = torch.randn(B, T, D, generator=g).bfloat16().float()
    w, b = 0.5 * torch.randn(W, D, generator=g), torch.randn(D, generator=g)
    y, dx, dw, db, ydt = _conv_gpu(x, w, b, go, torch.bfloat16, out_dtype=torch.bfloat16, strided=strided)
    assert ydt == torch.bfloat16
    wy = oconv.conv1d_fwd(x, w, b, compute=torch.float64)
    wdx, wdw, wdb = oconv.conv1d_bwd(x, w, go, compute=torch.float64)
    assert rel_l2(y, wy) <= BF16_TOL and rel_l2(dx, wdx) <= BF16_TOL
    assert rel_l2(dw, wdw) <= FP32_TOL * 10 and rel_l2(db, wdb) <= FP32_TOL * 10
    # bf16 storage only rounds the results: against the oracle rounded the same way they agree far closer
    assert rel_l2(y, wy.bfloat16().double()) <= 2e-3 and rel_l2(dx, wdx.bfloat16().double()) <= 2e-3


def test_conv_module_has_reference_parameters():
    from hawk_b200 import Conv1D
    m = Conv1D(width=64, temporal_width=4)
    assert [n for n, _ in m.named_parameters()] == ["w", "b"]
    assert m.w.shape == (4, 64) and m.b.shape == (64,) and m.w.dtype == torch.float32
    assert float(m.b.abs().max()) == 0.0 and abs(float(m.w.std()) - 0.05) < 0.02
    m = m.cuda()
    x = torch.randn(2, 10, 64, device="cuda")
    assert max_rel(m(x).cpu(), oconv.conv1d_fwd(x.cpu(), m.w.detach().cpu(), m.b.detach().cpu())) <= FP32_TOL
    assert torch.equal(m.doc_mask_forward(x), m(x))  # the reference's name for the same call (external.py:49,97-98)


@pytest.mark.parametrize("B,D", [(1, 64), (3, 72), (256, 2048)])
@pytest.mark.parametrize("dtype,sdtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                          (torch.float32, torch.bfloat16)])
def test_decode_steps_match_oracle(B, D, dtype, sdtype):
    from hawk_b200 import decode_conv_step, decode_rglru_step
    g = torch.Generator().manual_seed(B + D)
    rnd = lambda *s: torch.randn(*s, generator=g)
    xy = rnd(B, 2 * D).to(dtype)
    conv_state = rnd(B, 3, D).to(sdtype)
    w, b = rnd(4, D), rnd(D)
    lam = oscan.rnn_param_ring(D, generator=g)
    state = rnd(B, D).to(sdtype)
    # conv step on the strided x half
    cs = conv_state.cuda().clone()
    y = decode_conv_step(xy.cuda()[:, :D], cs, w.cuda(), b.cuda())
    wy, wcs = odec.conv_step(xy[:, :D].float(), conv_state.float(), w, b, compute=torch.float64)
    tol = FP32_TOL if dtype == torch.float32 else BF16_TOL
    assert y.dtype == dtype and rel_l2(y.float().cpu(), wy) <= tol
    assert torch.equal(cs.float().cpu(), wcs.float().to(sdtype).float())  # the roll is exact
    # recurrence step
    x, gx, ga = (rnd(B, D).to(dtype) for _ in range(3))
    st = state.cuda().clone()
    h = decode_rglru_step(x.cuda(), gx.cuda(), ga.cuda(), lam.cuda(), st)
    wh = odec.rglru_step(x.float(), gx.float(), ga.float(), lam, state.float(), compute=torch.float64)
    assert rel_l2(h.float().cpu(), wh) <= tol
    assert rel_l2(st.float().cpu(), wh) <= (FP32_TOL if sdtype == torch.float32 else BF16_TOL)


def test_decode_steps_reproduce_the_full_scan():
    """T cached steps equal the T-step training scan + conv (state carried in fp32)."""
    from hawk_b200 import decode_conv_step, decode_rglru_step, fused_linear_scan, temporal_conv1d
    g = torch.Generator().manual_seed(0)
    B, T, D = 4, 12, 128
    xin = torch.randn(B, T, D, generator=g).cuda()
    gx, ga = torch.randn(B, T, D, generator=g).cuda(), torch.randn(B, T, D, generator=g).cuda()
    w, b = torch.randn(4, D, generator=g).cuda(), torch.randn(D, generator=g).cuda()
    lam = oscan.rnn_param_ring(D, generator=g).cuda()
    xc = temporal_conv1d(xin, w, b)
    h = fused_linear_scan(xc, gx, ga, lam)
    cs = torch.zeros(B, 3, D, device="cuda")
    st = torch.zeros(B, D, device="cuda")
    for t in range(T):
        y = decode_conv_step(xin[:, t], cs, w, b)
        assert max_rel(y, xc[:, t]) <= FP32_TOL
        ht = decode_rglru_step(y, gx[:, t].contiguous(), ga[:, t].contiguous(), lam, st)
        assert max_rel(ht, h[:, t]) <= FP32_TOL


@pytest.mark.parametrize("B,R,nb", [(1, 64, 8), (3, 128, 16), (37, 512, 16), (256, 2048, 16), (20, 512, 4), (5, 6, 3)])
@pytest.mark.parametrize("dtype,sdtype,wdtype", [(torch.float32, torch.float32, torch.float32),
                                                 (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                                 (torch.bfloat16, torch.float32, torch.float32)])
def test_fused_decode_block_step_matches_oracle(B, R, nb, dtype, sdtype, wdtype):
    """conv step + both gate projections + RG-LRU step + gelu(y) * h in one launch == the oracle's
    statements of the four pieces chained (with the caches it leaves behind)."""
    import torch.nn.functional as F
    from hawk_b200 import ops
    from oracle import model as omodel
    g = torch.Generator().manual_seed(B + R + nb)
    rnd = lambda *s: torch.randn(*s, generator=g)
    bw = R // nb
    xy = rnd(B, 2 * R).to(dtype)
    conv_state, state = rnd(B, 3, R).to(sdtype), rnd(B, R).to(sdtype)
    cw, cb = 0.3 * rnd(4, R), 0.1 * rnd(R)
    wx, wa = ((rnd(nb, bw, bw) / bw ** 0.5).to(wdtype) for _ in range(2))
    bx, ba = 0.2 * rnd(nb, bw), 0.2 * rnd(nb, bw)
    lam = oscan.rnn_param_ring(R, generator=g)
    cs, st = conv_state.cuda().clone(), state.cuda().clone()
    out = ops.decode_block_step(xy.cuda(), cs, cw.cuda(), cb.cuda(), wx.cuda(), wa.cuda(), bx.cuda(), ba.cuda(),
                                lam.cuda(), st)
    d = torch.float64
    xc, wcs = odec.conv_step(xy[:, :R].float(), conv_state.float(), cw, cb, compute=d)
    gx = omodel.block_diag_linear(xc.to(d), wx.to(d), bx.to(d))
    ga = omodel.block_diag_linear(xc.to(d), wa.to(d), ba.to(d))
    wh = odec.rglru_step(xc.to(d), gx, ga, lam, state.float(), compute=d)
    want = F.gelu(xy[:, R:].to(d)) * wh
    tol = FP32_TOL if dtype == sdtype == torch.float32 else BF16_TOL
    assert out.dtype == dtype and out.shape == (B, R)
    assert rel_l2(out.float().cpu(), want) <= tol
    assert rel_l2(st.float().cpu(), wh) <= (FP32_TOL if sdtype == torch.float32 else BF16_TOL)
    assert torch.equal(cs.float().cpu(), wcs.float().to(sdtype).float())  # the roll is exact
