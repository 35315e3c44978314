"""Time-split scans (hawk_scan_fwd_split / hawk_scan_bwd_split): every sequence cut into sub-sequences that
run as separate CTAs, for launches with few (sequence, channel group) pairs.  The reference scans T in one
warp per channel block whatever the shape (hawk/scan_fused.py:83-109,199-260); the results must not depend
on how the time axis is cut.

Checked three ways: against the whole-sequence entry points on the same tensors (fp32 storage <= 1e-5,
bf16 storage within bf16 rounding), against the fp64 CPU oracle (1e-5 / 2e-2, norm-wise), and through the
public ops for shapes where the library chooses to split by itself.
"""
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_l2
from oracle import scan as oscan

pytestmark = pytest.mark.gpu

DT = {torch.float32: 0, torch.bfloat16: 1}


def _tensors(B, T, D, seed, dtype, gelu):
    g = torch.Generator().manual_seed(seed)
    x, gx, ga, go = (torch.randn(B, T, D, generator=g).to(dtype) for _ in range(4))
    xy = (torch.randn(B, T, 2 * D, generator=g) * 1.5).to(dtype) if gelu else None
    gb = 0.3 * torch.randn(2, D, generator=g)
    h0 = torch.randn(B, D, generator=g)
    lam = oscan.rnn_param_ring(D, generator=g)
    return x, gx, ga, go, xy, gb, h0, lam


def _run(t, nsub, use_h0, use_bias, gelu):
    """forward + backward through the C ABI; nsub = 0: whole-sequence entry points."""
    from hawk_b200 import _lib
    lib = _lib.load()
    x, gx, ga, go, xy, gb, h0, lam = (None if v is None else v.cuda() for v in t)
    B, T, D = x.shape
    dt = DT[x.dtype]
    st = torch.cuda.current_stream().cuda_stream
    p = lambda v: None if v is None else v.data_ptr()
    h0 = h0 if (use_h0 and not gelu) else None
    gb = gb if use_bias else None
    h, out = torch.empty_like(x), (torch.empty_like(x) if gelu else None)
    dx, dgx, dga = (torch.empty_like(x) for _ in range(3))
    dxy = torch.zeros_like(xy) if gelu else None
    y = xy[..., D:] if gelu else None
    dy = dxy[..., D:] if gelu else None
    dlam = torch.empty(D, device="cuda")
    dh0 = torch.empty(B, D, device="cuda") if not gelu else None
    dgb = torch.empty(2, D, device="cuda") if use_bias else None
    ys = (y.stride(0), y.stride(1)) if gelu else (0, 0)
    if nsub:
        ws = torch.empty(lib.hawk_scan_split_workspace_bytes(B, nsub, D), dtype=torch.uint8, device="cuda")
        _lib.check(lib.hawk_scan_fwd_split(p(x), p(gx), p(ga), p(lam), p(h0), p(gb), p(y), ys[0], ys[1], p(h), p(out), nsub,
                                           p(ws), ws.numel(), B, T, D, dt, st), "fwd_split")
        _lib.check(lib.hawk_scan_bwd_split(p(x), p(gx), p(ga), p(lam), p(h0), p(gb), p(h), p(y), ys[0], ys[1], p(go), p(dx),
                                           p(dgx), p(dga), p(dy), ys[0], ys[1], p(dlam), p(dh0), p(dgb), nsub, p(ws),
                                           ws.numel(), B, T, D, dt, st), "bwd_split")
    else:
        ws = torch.empty(lib.hawk_scan_bwd_workspace_bytes(B, D), dtype=torch.uint8, device="cuda")
        if gelu:
            _lib.check(lib.hawk_scan_gelu_fwd(p(x), p(gx), p(ga), p(lam), p(gb), p(y), ys[0], ys[1], p(h), p(out), B, T, D,
                                              dt, st), "gelu_fwd")
            _lib.check(lib.hawk_scan_gelu_bwd(p(x), p(gx), p(ga), p(lam), p(gb), p(h), p(y), ys[0], ys[1], p(go), p(dx),
                                              p(dgx), p(dga), p(dy), ys[0], ys[1], p(dlam), p(dgb), p(ws), ws.numel(), B, T,
                                              D, dt, st), "gelu_bwd")
        else:
            _lib.check(lib.hawk_scan_fwd(p(x), p(gx), p(ga), p(lam), p(h0), p(gb), p(h), B, T, D, dt, st), "fwd")
            _lib.check(lib.hawk_scan_bwd(p(x), p(gx), p(ga), p(lam), p(h0), p(gb), p(h), p(go), p(dx), p(dgx), p(dga),
                                         p(dlam), p(dh0), p(dgb), p(ws), ws.numel(), B, T, D, dt, st), "bwd")
    torch.cuda.synchronize()
    res = dict(h=h, dx=dx, dgx=dgx, dga=dga, dlam=dlam)
    if gelu:
        res.update(out=out, dy=dy)
        assert float(dxy[..., :D].abs().max()) == 0.0
    else:
        res["dh0"] = dh0
    if use_bias:
        res["dgb"] = dgb
    return {k: v.float().cpu() for k, v in res.items()}


def _oracle(t, use_h0, use_bias, gelu):
    """fp64 autograd through a differentiable statement of the recurrence (hawk/scan_fused.py:44-109 forward),
    extended with the initial state, the gate biases and the gelu(y) * h epilogue (hawk/hawk.py:134-135)."""
    x, gx, ga, go, xy, gb, h0, lam = t
    B, T, D = x.shape
    leaves = dict(x=x, gx=gx, ga=ga, lam=lam)
    if use_bias:
        leaves["gb"] = gb
    if use_h0 and not gelu:
        leaves["h0"] = h0
    if gelu:
        leaves["y"] = xy[..., D:]
    L = {k: v.float().double().requires_grad_(True) for k, v in leaves.items()}
    bx, ba = (L["gb"][0], L["gb"][1]) if use_bias else (0.0, 0.0)
    a = torch.exp(-8.0 * torch.sigmoid(L["ga"] + ba) * F.softplus(L["lam"]))
    beta = L["x"] * torch.sigmoid(L["gx"] + bx) * torch.sqrt(1 - a * a)
    st = L["h0"] if "h0" in L else torch.zeros(B, D, dtype=torch.float64)
    hs = []
    for k in range(T):
        st = a[:, k] * st + beta[:, k]
        hs.append(st)
    h = torch.stack(hs, 1)
    res = F.gelu(L["y"]) * h if gelu else h
    grads = torch.autograd.grad(res, list(L.values()), go.float().double())
    want = dict(h=h.detach())
    if gelu:
        want["out"] = res.detach()
    names = dict(x="dx", gx="dgx", ga="dga", lam="dlam", gb="dgb", h0="dh0", y="dy")
    for k, g in zip(L.keys(), grads):
        want[names[k]] = g
    return want


CASES = [  # B, T, D, nsub
    (1, 512, 64, 2), (1, 1024, 128, 4), (2, 990, 64, 3), (1, 2310, 192, 7), (3, 768, 64, 6), (1, 4096, 128, 16),
    (1, 65, 64, 5), (2, 7, 64, 7),
]


@pytest.mark.parametrize("gelu", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,T,D,nsub", CASES)
def test_split_matches_whole_sequence_and_oracle(B, T, D, nsub, dtype, gelu):
    use_h0, use_bias = (T % 2 == 0), (B % 2 == 1)
    t = _tensors(B, T, D, seed=T + D + nsub, dtype=dtype, gelu=gelu)
    whole = _run(t, 0, use_h0, use_bias, gelu)
    split = _run(t, nsub, use_h0, use_bias, gelu)
    # the two differ only by how the fp32 recurrence is associated (and, in bf16, by last-bit roundings of h
    # that the backward then reads)
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    for k in whole:
        assert rel_l2(split[k], whole[k]) <= tol, (k, rel_l2(split[k], whole[k]))
    otol = 1e-5 if dtype == torch.float32 else 2e-2
    want = _oracle(t, use_h0, use_bias, gelu)
    for k, v in want.items():
        assert rel_l2(split[k], v) <= otol, (k, rel_l2(split[k], v))


def test_split_rejects_bad_arguments():
    from hawk_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(1, 100, 64, device="cuda")
    h = torch.empty_like(x)
    lam = torch.zeros(64, device="cuda")
    ws = torch.empty(lib.hawk_scan_split_workspace_bytes(1, 4, 64), dtype=torch.uint8, device="cuda")
    p = lambda v: v.data_ptr()
    call = lambda nsub, wsb: lib.hawk_scan_fwd_split(p(x), p(x), p(x), p(lam), None, None, None, 0, 0, p(h), None, nsub,
                                                     p(ws), wsb, 1, 100, 64, 0, None)
    assert call(3, ws.numel()) != 0       # 100 rows do not split in three
    assert call(65, ws.numel()) != 0      # more sub-sequences than supported
    assert call(4, ws.numel() - 1) != 0   # workspace too small
    assert call(4, ws.numel()) == 0
    torch.cuda.synchronize()


def test_library_chooses_to_split_small_launches():
    from hawk_b200 import _lib
    lib = _lib.load()
    FWD, FWD_GELU, BWD = 0, 1, 2
    for which in (FWD, FWD_GELU, BWD):
        assert lib.hawk_scan_split_chunks(8, 4096, 2048, which) == 1       # the benchmark's shape: 512 CTAs already
        assert lib.hawk_scan_split_chunks(1, 65536, 4096, which) == 1      # 128+ CTAs: reading twice would cost more
        n = lib.hawk_scan_split_chunks(1, 65536, 512, which)
        assert n > 1 and 65536 % n == 0 and 65536 // n >= 256
        assert lib.hawk_scan_split_chunks(1, 1021, 512, which) == 1        # a prime number of rows cannot be cut evenly
    for T in (65536, 4096, 300, 255):  # whatever the shape, the answer is one the split entry points accept
        n = lib.hawk_scan_split_chunks(1, T, 64, BWD)
        assert 1 <= n <= 64 and T % n == 0 and (n == 1 or T // n >= 256)
    # 64 CTAs of 32 channels: the backward and the fused forward split, the plain forward (128 CTAs of 16) does not
    assert lib.hawk_scan_split_chunks(1, 65536, 2048, FWD) == 1
    assert lib.hawk_scan_split_chunks(1, 65536, 2048, FWD_GELU) > 1 and lib.hawk_scan_split_chunks(1, 65536, 2048, BWD) > 1


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_public_ops_split_long_narrow_sequences(dtype, tol):
    """B=1, T=4096, D=256 (8 channel groups): fused_linear_scan and fused_scan_gelu take the split path
    (the launch log names it) and agree with the fp64 oracle."""
    from hawk_b200 import fused_linear_scan, fused_scan_gelu, ops
    B, T, D = 1, 4096, 256
    t = _tensors(B, T, D, seed=11, dtype=dtype, gelu=True)
    x, gx, ga, go, xy, gb, h0, lam = t
    dev = "cuda"
    leaves = [v.to(dev).requires_grad_(True) for v in (x, gx, ga)]
    lam_d, gb_d, xy_d = lam.to(dev).requires_grad_(True), gb.to(dev).requires_grad_(True), xy.to(dev).requires_grad_(True)
    ops.LOG.reset()
    try:
        out, h = fused_scan_gelu(*leaves, lam_d, xy_d[..., D:], gate_bias=gb_d)
        out.backward(go.to(dev))
        counts = dict(ops.LOG.counts)
    finally:
        ops.LOG.reset(enabled=False)
    assert counts.get("scan_gelu_fwd_split") == 3 and counts.get("scan_gelu_bwd_split") == 5, counts
    got = dict(h=h.detach(), out=out.detach(), dx=leaves[0].grad, dgx=leaves[1].grad, dga=leaves[2].grad, dlam=lam_d.grad,
               dy=xy_d.grad[..., D:], dgb=gb_d.grad)
    got = {k: v.float().cpu() for k, v in got.items()}
    want = _oracle(t, False, True, True)
    for k, v in want.items():
        assert rel_l2(got[k], v) <= tol, (k, rel_l2(got[k], v))
    # plain scan with an initial state
    leaves = [v.to(dev).requires_grad_(True) for v in (x, gx, ga)]
    h0_d = h0.to(dev).requires_grad_(True)
    lam_d = lam.to(dev).requires_grad_(True)
    hh = fused_linear_scan(*leaves, lam_d, h0=h0_d)
    hh.backward(go.to(dev))
    got = dict(h=hh.detach(), dx=leaves[0].grad, dgx=leaves[1].grad, dga=leaves[2].grad, dlam=lam_d.grad, dh0=h0_d.grad)
    got = {k: v.float().cpu() for k, v in got.items()}
    want = _oracle(t, True, False, False)
    for k, v in want.items():
        assert rel_l2(got[k], v) <= tol, (k, rel_l2(got[k], v))
