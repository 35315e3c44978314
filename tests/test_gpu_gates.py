"""The fused block-diagonal gate projections (hawk_gates_fwd / hawk_gates_bwd, through the C ABI) against the
CPU oracle `oracle.model.block_diag_linear` (hawk/external.py:224-233) in fp64 on the same bf16-rounded
operands; gradients from autograd of the oracle.  The kernels multiply bf16 operands with fp32
accumulation and store bf16 (what the reference's einsum does under autocast): bound 2e-2, norm-wise.
"""
import pytest
import torch

from conftest import max_rel, rel_l2
from oracle import model as omodel

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _case(M, nb, bw, seed):
    g = torch.Generator().manual_seed(seed)
    R = nb * bw
    bf = lambda t: t.to(torch.bfloat16)
    xc = bf(torch.randn(M, R, generator=g))
    wx = bf(torch.randn(nb, bw, bw, generator=g) / bw ** 0.5)
    wa = bf(torch.randn(nb, bw, bw, generator=g) / bw ** 0.5)
    dgx, dga, dxc0 = (bf(torch.randn(M, R, generator=g)) for _ in range(3))
    return xc, wx, wa, dgx, dga, dxc0


def _oracle(xc, wx, wa, dgx, dga, dxc0):
    x = xc.double().requires_grad_(True)
    wxd, wad = wx.double().requires_grad_(True), wa.double().requires_grad_(True)
    zero = torch.zeros(wx.shape[0], wx.shape[1], dtype=torch.float64)
    gx = omodel.block_diag_linear(x, wxd, zero)
    ga = omodel.block_diag_linear(x, wad, zero)
    (gx * dgx.double()).sum().add((ga * dga.double()).sum()).backward()
    return gx.detach(), ga.detach(), dxc0.double() + x.grad, wxd.grad, wad.grad


SHAPES = [(256, 16, 128), (1000, 16, 32), (300, 4, 64), (389, 2, 128), (77, 8, 16), (128, 1, 128), (5000, 16, 128)]


@pytest.mark.parametrize("M,nb,bw", SHAPES)
@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
def test_fused_gates_match_oracle(M, nb, bw, w_dtype):
    from hawk_b200 import ops
    xc, wx, wa, dgx, dga, dxc0 = _case(M, nb, bw, seed=M + nb + bw)
    want = _oracle(xc, wx, wa, dgx, dga, dxc0)
    dev = "cuda:0"
    assert ops.gates_kernel_ok(xc.to(dev), nb, bw)
    packed = ops.gates_pack(wx.to(dev, w_dtype), wa.to(dev, w_dtype))
    out = ops.gates_fwd(xc.to(dev), packed, bw)
    dxc = dxc0.to(dev).clone()
    dwx, dwa = ops.gates_bwd_into(xc.to(dev), dgx.to(dev), dga.to(dev), packed, dxc, bw)
    ops.check_device_status()
    got = (out[0], out[1], dxc, dwx, dwa)
    for name, a, b in zip(("gx", "ga", "dxc", "dwx", "dwa"), got, want):
        assert a.shape == b.shape, name
        assert rel_l2(a.float().cpu(), b) <= TOL, (name, rel_l2(a.float().cpu(), b))
        assert max_rel(a.float().cpu(), b) <= TOL, (name, max_rel(a.float().cpu(), b))


def test_fused_gates_autograd_equals_strided_batch_form():
    """fused_block_diag_gates (tcgen05) against block_diag_gates (cuBLAS strided batch) on the same tensors."""
    from hawk_b200 import ops
    xc, wx, wa, dgx, dga, _ = _case(2048, 16, 128, seed=3)
    dev = "cuda:0"
    res = []
    for fn in (lambda x, a, b: ops.fused_block_diag_gates(x, a, b), lambda x, a, b: ops.block_diag_gates(x, a, None, b, None)):
        x = xc.to(dev).view(2, 1024, 2048).requires_grad_(True)
        a, b = wx.to(dev).float().requires_grad_(True), wa.to(dev).float().requires_grad_(True)
        gx, ga = fn(x, a, b)
        torch.autograd.backward((gx, ga), (dgx.to(dev).view_as(gx), dga.to(dev).view_as(ga)))
        res.append((gx.detach(), ga.detach(), x.grad, a.grad, b.grad))
    for name, p, q in zip(("gx", "ga", "dx", "dwx", "dwa"), *res):
        assert rel_l2(p.float(), q.float()) <= 8e-3, (name, rel_l2(p.float(), q.float()))


def test_fused_gates_training_shape_weight_gradient():
    """M = 8 * 4096 rows, R = 2048, 16 blocks of 128 (the 1.35 B model's shape): the weight gradient contracts
    over all 32768 rows in 9 splits; checked in full against fp32 CPU einsum, forward on sampled rows."""
    from hawk_b200 import ops
    M, nb, bw = 32768, 16, 128
    xc, wx, wa, dgx, dga, dxc0 = _case(M, nb, bw, seed=9)
    dev = "cuda:0"
    packed = ops.gates_pack(wx.to(dev), wa.to(dev))
    out = ops.gates_fwd(xc.to(dev), packed, bw)
    dxc = torch.zeros(M, nb * bw, dtype=torch.bfloat16, device=dev)
    dwx, dwa = ops.gates_bwd_into(xc.to(dev), dgx.to(dev), dga.to(dev), packed, dxc, bw)
    ops.check_device_status()
    xs = xc.float().view(M, nb, bw)
    want_dwx = torch.einsum("mhi,mhj->hij", xs, dgx.float().view(M, nb, bw))
    want_dwa = torch.einsum("mhi,mhj->hij", xs, dga.float().view(M, nb, bw))
    assert rel_l2(dwx.cpu(), want_dwx) <= 1e-3 and rel_l2(dwa.cpu(), want_dwa) <= 1e-3
    rows = torch.arange(0, M, 331)
    want_gx = torch.einsum("mhi,hij->mhj", xs[rows].double(), wx.double()).reshape(len(rows), -1)
    assert rel_l2(out[0][rows].float().cpu(), want_gx) <= TOL
    want_dx = (torch.einsum("mhj,hij->mhi", dgx.float().view(M, nb, bw)[rows].double(), wx.double()) +
               torch.einsum("mhj,hij->mhi", dga.float().view(M, nb, bw)[rows].double(), wa.double())).reshape(len(rows), -1)
    assert rel_l2(dxc[rows].float().cpu(), want_dx) <= TOL


def test_device_side_wait_gives_up_and_reports():
    """A tcgen05 kernel whose TMA producer never delivers must not hang: with a wait budget of 1e5 cycles the
    kernel returns by itself and sets the status word; the context stays usable."""
    from hawk_b200 import _lib, ops
    lib = _lib.load()
    dev = torch.device("cuda:0")
    scratch = torch.zeros(262144, dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.hawk_debug_wait_timeout(scratch.data_ptr(), scratch.numel(), 100000, status.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    # and real work still runs afterwards
    xc, wx, wa, *_ = _case(128, 1, 128, seed=1)
    out = ops.gates_fwd(xc.to(dev), ops.gates_pack(wx.to(dev), wa.to(dev)), 128)
    ops.check_device_status()
    want = omodel.block_diag_linear(xc.double(), wx.double(), torch.zeros(1, 128, dtype=torch.float64))
    assert rel_l2(out[0].float().cpu(), want) <= TOL
