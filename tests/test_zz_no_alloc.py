"""hawk_scan_bwd_noalloc: the scan backward for hosts that are not allowed to allocate device memory
while running (all memory handed to their own arena at start-up, or a loop that cannot take
cudaMalloc's device-wide synchronisation).  Its [B,D] scratch is a fixed array inside the library.

Called here straight through the C ABI and compared with hawk_scan_bwd on two calls in a row with
different inputs and shapes, so that anything the first call leaves in the shared array would show
up in the second.  Collected last on purpose (file name), and also passes alone in a fresh process."""
import ctypes

import pytest
import torch

from conftest import max_rel, rel_l2

pytestmark = pytest.mark.gpu


def _both(lib, B, T, D, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x, gx, ga, go = (torch.randn(B, T, D, generator=g, device="cuda").to(dtype) for _ in range(4))
    lam = (torch.rand(D, generator=g, device="cuda") * 4.0 - 6.5).contiguous()
    code = 1 if dtype == torch.bfloat16 else 0
    stream = torch.cuda.current_stream().cuda_stream
    h = torch.empty_like(x)
    assert lib.hawk_scan_fwd(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(), None, None,
                             h.data_ptr(), B, T, D, code, stream) == 0

    def outs():
        return [torch.empty_like(x) for _ in range(3)] + [torch.empty(D, device="cuda"), torch.empty(B, D, device="cuda")]

    ref = outs()
    ws_bytes = lib.hawk_scan_bwd_workspace_bytes(B, D)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    rc = lib.hawk_scan_bwd(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(), None, None, h.data_ptr(),
                           go.data_ptr(), *[t.data_ptr() for t in ref], None, ws.data_ptr(), ws_bytes, B, T, D, code, stream)
    assert rc == 0
    got = outs()  # the caller still provides inputs and outputs; only the scratch is built in
    rc = lib.hawk_scan_bwd_noalloc(x.data_ptr(), gx.data_ptr(), ga.data_ptr(), lam.data_ptr(), None, h.data_ptr(),
                                   go.data_ptr(), *[t.data_ptr() for t in got], B, T, D, code, stream)
    assert rc == 0, lib.hawk_strerror(rc)
    torch.cuda.synchronize()
    return got, ref


def test_noalloc_backward_equals_workspace_backward_twice_in_a_row():
    import hawk_b200._lib as L
    lib = L.load()
    tol = {torch.float32: 1e-5, torch.bfloat16: 2e-2}
    # second call: other shape, other values, fewer (batch x channel) entries than the first left behind
    for (B, T, D, dtype, seed) in [(4, 300, 256, torch.bfloat16, 1), (2, 77, 128, torch.float32, 2)]:
        got, ref = _both(lib, B, T, D, dtype, seed)
        for name, a, b in zip(("dx", "dgx", "dga", "dlam", "dh0"), got, ref):
            assert torch.isfinite(a.float()).all(), name
            assert rel_l2(a.float().cpu(), b.float().cpu()) <= tol[dtype], name
            assert max_rel(a.float().cpu(), b.float().cpu()) <= tol[dtype], name


def test_noalloc_rejects_sizes_beyond_its_scratch():
    import hawk_b200._lib as L
    lib = L.load()
    p = ctypes.c_void_p(4096)  # never dereferenced: the size check comes first
    rc = lib.hawk_scan_bwd_noalloc(p, p, p, p, None, p, p, p, p, p, p, None, 129, 8, 2048, 1, None)  # 264192 > 262144
    assert rc == -9
    assert b"262144" in lib.hawk_strerror(rc)
