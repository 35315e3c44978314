"""torch.compile(fullgraph=True) traces the model shell and the fused operators as ONE graph: no graph break
inside this library's custom ops or autograd Functions.  Tracing runs on fake tensors, so no GPU is needed;
the compiler backend used here stops after receiving the graph (nothing is executed)."""
import pytest
import torch
import torch._dynamo


class _Traced(Exception):
    pass


def _trace(fn, *args):
    graphs = []

    def backend(gm, example_inputs):
        graphs.append(gm)
        raise _Traced()

    torch._dynamo.reset()
    try:
        torch.compile(fn, fullgraph=True, backend=backend)(*args)
    except Exception as e:  # noqa: BLE001
        chain, seen = e, []
        while chain is not None and not isinstance(chain, _Traced):
            seen.append(chain)
            chain = chain.__cause__ or chain.__context__
        if chain is None and "_Traced" not in repr(seen):
            raise
    assert len(graphs) == 1, "the function was split into several graphs"
    return [str(n.target) for n in graphs[0].graph.nodes if n.op == "call_function"]


def test_model_forward_is_one_graph():
    import hawk_b200.model as M
    model = M.HawkModel(M.HawkConfig(96, 64, 128, 2, 64, 4, 4))
    ids = torch.randint(1, 96, (2, 17))
    targets = _trace(model, ids, ids)
    assert sum("autograd_function_apply" in t for t in targets) == 2  # one recurrent core per layer
    assert any("linear_ce" in t for t in targets) and any("add_rms_norm_fwd" in t for t in targets)


def test_fused_operator_functions_trace(monkeypatch):
    from hawk_b200 import ops
    xy = torch.randn(2, 16, 256, dtype=torch.bfloat16, requires_grad=True)
    cw, cb = torch.randn(4, 128), torch.zeros(128)
    wx, wa = torch.randn(1, 128, 128), torch.randn(1, 128, 128)
    gb, lam = torch.zeros(2, 128), torch.randn(128)
    x = torch.randn(4, 8, 64, requires_grad=True)
    w = torch.randn(32, 64, requires_grad=True)
    _trace(lambda a, b: ops._AutocastLinear.apply(a, b, None).sum(), x, w)
    _trace(lambda a: ops.fused_scan_gelu(a[..., :128], a[..., :128], a[..., :128], lam, a[..., 128:])[0].float().sum(), xy)
    _trace(lambda a: ops._FusedGates.apply(a[..., :128], wx, wa)[0].float().sum(), xy)
    for fused in (False, True):  # the recurrent core with the cuBLAS form and with the fused gate kernels
        monkeypatch.setattr(ops, "gates_kernel_ok", lambda x_, nb, bw, f=fused: f)
        _trace(lambda a: ops.recurrent_core(a, cw, cb, wx, wa, gb, lam)[0].float().sum(), xy)
