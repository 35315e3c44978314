"""Out-of-bounds check without a sanitizer: every output (and workspace) handed to the C ABI sits inside
a larger buffer filled with a canary pattern; after the call the guard zones must be untouched.
Shapes with ragged time tails and the smallest legal widths exercise the predicated paths."""
import pytest
import torch

pytestmark = pytest.mark.gpu
PAD = 4096  # elements on either side (keeps 16-byte alignment for every dtype used)


class Guarded:
    def __init__(self, shape, dtype, fill=None):
        n = 1
        for s in shape:
            n *= s
        self.n = n
        canary = 1024.0 if dtype != torch.uint8 else 0xA5
        self.canary = canary
        self.buf = torch.full((n + 2 * PAD,), canary, dtype=dtype, device="cuda")
        self.t = self.buf[PAD:PAD + n].view(shape)
        if fill is not None:
            self.t.copy_(fill)

    def intact(self):
        return bool((self.buf[:PAD] == self.canary).all()) and bool((self.buf[PAD + self.n:] == self.canary).all())


def _lib():
    import hawk_b200._lib as L
    return L.load()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,T,D", [(1, 1, 64), (2, 33, 64), (3, 129, 128), (1, 1027, 192)])
def test_scan_writes_stay_in_bounds(dtype, B, T, D):
    lib = _lib()
    code = 1 if dtype == torch.bfloat16 else 0
    g = torch.Generator(device="cuda").manual_seed(B + T + D)
    x, gx, ga, go = (Guarded((B, T, D), dtype, torch.randn(B, T, D, generator=g, device="cuda")) for _ in range(4))
    lam = torch.rand(D, device="cuda") * 4 - 6
    h, dx, dgx, dga = (Guarded((B, T, D), dtype) for _ in range(4))
    dlam, dh0 = Guarded((D,), torch.float32), Guarded((B, D), torch.float32)
    gb = Guarded((2, D), torch.float32, torch.randn(2, D, generator=g, device="cuda"))
    dgb = Guarded((2, D), torch.float32)
    ws_bytes = lib.hawk_scan_bwd_workspace_bytes(B, D)
    ws = Guarded((ws_bytes,), torch.uint8)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.hawk_scan_fwd(x.t.data_ptr(), gx.t.data_ptr(), ga.t.data_ptr(), lam.data_ptr(), None, gb.t.data_ptr(),
                             h.t.data_ptr(), B, T, D, code, st) == 0
    assert lib.hawk_scan_bwd(x.t.data_ptr(), gx.t.data_ptr(), ga.t.data_ptr(), lam.data_ptr(), None, gb.t.data_ptr(),
                             h.t.data_ptr(), go.t.data_ptr(), dx.t.data_ptr(), dgx.t.data_ptr(), dga.t.data_ptr(),
                             dlam.t.data_ptr(), dh0.t.data_ptr(), dgb.t.data_ptr(), ws.t.data_ptr(), ws_bytes,
                             B, T, D, code, st) == 0
    torch.cuda.synchronize()
    for name, gd in dict(x=x, gx=gx, ga=ga, go=go, h=h, dx=dx, dgx=dgx, dga=dga, dlam=dlam, dh0=dh0, gb=gb, dgb=dgb,
                         ws=ws).items():
        assert gd.intact(), name
    for gd in (h, dx, dgx, dga, dlam, dh0, dgb):  # and every element inside was written
        assert bool((gd.t.float() != 1024.0).all()) and bool(torch.isfinite(gd.t.float()).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,T,D,W", [(1, 1, 8, 4), (2, 3, 8, 4), (2, 65, 24, 3), (3, 513, 72, 4)])
def test_conv_writes_stay_in_bounds(dtype, B, T, D, W):
    lib = _lib()
    code = 1 if dtype == torch.bfloat16 else 0
    g = torch.Generator(device="cuda").manual_seed(T + D)
    x = Guarded((B, T, D), dtype, torch.randn(B, T, D, generator=g, device="cuda"))
    go = Guarded((B, T, D), dtype, torch.randn(B, T, D, generator=g, device="cuda"))
    w, b = torch.randn(W, D, device="cuda"), torch.randn(D, device="cuda")
    y, dx = Guarded((B, T, D), dtype), Guarded((B, T, D), dtype)
    dw, db = Guarded((W, D), torch.float32), Guarded((D,), torch.float32)
    ws_bytes = lib.hawk_conv1d_bwd_workspace_bytes(B, T, D, W)
    ws = Guarded((ws_bytes,), torch.uint8)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.hawk_conv1d_fwd(x.t.data_ptr(), T * D, D, w.data_ptr(), b.data_ptr(), y.t.data_ptr(), B, T, D, W,
                               code, code, st) == 0
    assert lib.hawk_conv1d_bwd(go.t.data_ptr(), x.t.data_ptr(), T * D, D, w.data_ptr(), dx.t.data_ptr(), T * D, D,
                               dw.t.data_ptr(), db.t.data_ptr(), ws.t.data_ptr(), ws_bytes, B, T, D, W, code, code,
                               st) == 0
    torch.cuda.synchronize()
    for name, gd in dict(x=x, go=go, y=y, dx=dx, dw=dw, db=db, ws=ws).items():
        assert gd.intact(), name
    for gd in (y, dx, dw, db):
        assert bool((gd.t.float() != 1024.0).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,J", [(1, 8), (5, 24), (1001, 64), (3, 256), (595, 128)])
def test_glue_writes_stay_in_bounds(dtype, M, J):
    lib = _lib()
    code = 1 if dtype == torch.bfloat16 else 0
    H = 8 * J  # rms_norm width
    g = torch.Generator(device="cuda").manual_seed(M + J)
    a = Guarded((M, J), dtype, torch.randn(M, J, generator=g, device="cuda"))
    b = Guarded((M, J), dtype, torch.randn(M, J, generator=g, device="cuda"))
    out, da, db = (Guarded((M, J), dtype) for _ in range(3))
    st = torch.cuda.current_stream().cuda_stream
    assert lib.hawk_gelu_mul_fwd(a.t.data_ptr(), J, b.t.data_ptr(), J, out.t.data_ptr(), J, M, J, code, st) == 0
    assert lib.hawk_gelu_mul_bwd(out.t.data_ptr(), J, a.t.data_ptr(), J, b.t.data_ptr(), J, da.t.data_ptr(), J,
                                 db.t.data_ptr(), J, M, J, code, st) == 0
    x = Guarded((M, H), torch.float32, torch.randn(M, H, generator=g, device="cuda"))
    delta = Guarded((M, H), dtype, torch.randn(M, H, generator=g, device="cuda"))
    w = torch.ones(H, device="cuda")
    xo, dx = Guarded((M, H), torch.float32), Guarded((M, H), torch.float32)
    y, dd = Guarded((M, H), dtype), Guarded((M, H), dtype)
    rstd, dw = Guarded((M,), torch.float32), Guarded((H,), torch.float32)
    ws_bytes = lib.hawk_rms_norm_bwd_workspace_bytes(H)
    ws = Guarded((ws_bytes,), torch.uint8)
    assert lib.hawk_add_rms_norm_fwd(x.t.data_ptr(), delta.t.data_ptr(), xo.t.data_ptr(), w.data_ptr(), y.t.data_ptr(),
                                     rstd.t.data_ptr(), M, H, 1e-6, 0, code, st) == 0
    assert lib.hawk_add_rms_norm_bwd(y.t.data_ptr(), xo.t.data_ptr(), w.data_ptr(), rstd.t.data_ptr(), x.t.data_ptr(),
                                     dx.t.data_ptr(), dd.t.data_ptr(), dw.t.data_ptr(), ws.t.data_ptr(), ws_bytes, M, H,
                                     0, code, st) == 0
    torch.cuda.synchronize()
    for name, gd in dict(a=a, b=b, out=out, da=da, db=db, x=x, delta=delta, xo=xo, dx=dx, y=y, dd=dd, rstd=rstd,
                         dw=dw, ws=ws).items():
        assert gd.intact(), name
    for gd in (out, da, db, xo, dx, y, dd, rstd, dw):
        assert bool((gd.t.float() != 1024.0).all())
