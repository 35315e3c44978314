"""The training harness's own pieces on the GPU: the fused AdamW kernel against torch.optim.AdamW, and the
bf16 weight copies it hands to the model's Linear layers."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _params(sizes, misaligned=False):
    g = torch.Generator().manual_seed(11)
    out = []
    for n in sizes:
        if misaligned:  # a contiguous view that starts 4 bytes into its allocation: the kernel's scalar path
            base = torch.randn(n + 1, generator=g).cuda()
            out.append(torch.nn.Parameter(base[1:]))
        else:
            out.append(torch.nn.Parameter(torch.randn(n, generator=g).cuda()))
    return out


@pytest.mark.parametrize("misaligned", [False, True])
def test_fused_adamw_matches_torch_adamw(misaligned):
    from hawk_b200.train import FusedAdamW
    sizes = [1, 7, 4096, 100003, (1 << 20) + 2]
    mine, ref = _params(sizes, misaligned), _params(sizes, misaligned)
    kw = dict(lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    o1, o2 = FusedAdamW(mine, **kw), torch.optim.AdamW(ref, foreach=False, fused=False, **kw)
    g = torch.Generator(device="cuda").manual_seed(5)
    for step in range(6):
        for a, b in zip(mine, ref):
            gr = torch.randn(a.shape, generator=g, device="cuda") * (10.0 ** (step - 3))
            a.grad, b.grad = gr.clone(), gr.clone()
        v0 = [a._version for a in mine]
        o1.step()
        o2.step()
        assert all(a._version > v for a, v in zip(mine, v0))  # autograd sees the in-place update
        for a, b in zip(mine, ref):
            assert float((a - b).abs().max()) <= 2e-6 * float(b.abs().max()), step
    # state round trip: a fresh optimiser loaded from the state dict continues identically
    o3 = FusedAdamW(mine, **kw)
    o3.load_state_dict(o1.state_dict())
    assert all(not k.startswith("_") for st in o1.state_dict()["state"].values() for k in st)
    for a, b in zip(mine, ref):
        gr = torch.randn(a.shape, generator=g, device="cuda")
        a.grad, b.grad = gr.clone(), gr.clone()
    o3.step()
    o2.step()
    for a, b in zip(mine, ref):
        assert float((a - b).abs().max()) <= 2e-6 * float(b.abs().max())
    o1 = o3
    for a, b in zip(mine, ref):
        sa, sb = o1.state[a], o2.state[b]
        assert float((sa["exp_avg"] - sb["exp_avg"]).abs().max()) <= 1e-6 * float(sb["exp_avg"].abs().max())
        assert float((sa["exp_avg_sq"] - sb["exp_avg_sq"]).abs().max()) <= 1e-6 * float(sb["exp_avg_sq"].abs().max())


def test_trainer_keeps_bf16_weight_copies_current():
    import hawk_b200.model as M
    from hawk_b200 import train
    cfg = M.HawkConfig(300, 128, 256, 2, 128, 16, 4)
    tr = train.Trainer(cfg, "cuda", seed=0, lr=1e-3)
    lins = [m for m in tr.model.modules() if isinstance(m, M.Linear)]
    assert len(lins) == 8 and all(m.weight_bf16 is None for m in lins)
    ids = torch.randint(1, 300, (4, 64), device="cuda")
    l0 = float(tr.step(ids))
    for m in lins:  # written by the optimiser kernel, bit-identical to a cast of the updated weight
        assert m.weight_bf16_version == m.weight._version
        assert torch.equal(m.weight_bf16, m.weight.detach().to(torch.bfloat16))
    losses = [float(tr.step(ids)) for _ in range(5)]
    assert min(losses) < l0
    # a weight changed behind the optimiser's back (load_state_dict, manual edits) invalidates its copy
    m = lins[0]
    with torch.no_grad():
        m.weight.mul_(0.5)
    assert m.weight_bf16_version != m.weight._version
    x = torch.randn(3, m.in_features, device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m(x)
        want = torch.nn.functional.linear(x, m.weight)
    assert torch.equal(y, want)
    # a write through .data is invisible to the version counter: the documented remedy is drop_bf16_copies
    tr.step(ids)
    with torch.no_grad():
        m.weight.data.mul_(2.0)
    assert m.weight_bf16_version == m.weight._version  # the stale copy would be used ...
    M.drop_bf16_copies(tr.model)
    assert m.weight_bf16 is None
    with torch.autocast("cuda", dtype=torch.bfloat16):
        assert torch.equal(m(x), torch.nn.functional.linear(x, m.weight))  # ... not after dropping it
