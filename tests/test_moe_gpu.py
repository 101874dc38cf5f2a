"""Mixture-of-experts kernels against the fp32 PyTorch statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("cfg", [
    dict(E=128, k=8, scoring="softmax", norm=True, groups=(1, 1), bias=False, scale=1.0),
    dict(E=64, k=6, scoring="sigmoid", norm=True, groups=(8, 4), bias=True, scale=2.446),
    dict(E=8, k=2, scoring="softmax", norm=False, groups=(1, 1), bias=False, scale=1.0),
    dict(E=256, k=8, scoring="sigmoid", norm=True, groups=(8, 4), bias=False, scale=2.5),
])
def test_router_matches_reference(cfg):
    from chatlearn_b200 import ops
    from chatlearn_b200.ops import reference as ref
    torch.manual_seed(0)
    T, E, k = 333, cfg["E"], cfg["k"]
    logits = torch.randn(T, E, device=_dev()) * 2
    bias = torch.randn(E, device=_dev()) * 0.1 if cfg["bias"] else None
    a = logits.clone().requires_grad_(True)
    b = logits.clone().requires_grad_(True)
    w1, i1, s1 = ops.moe_router(a, k, cfg["scoring"], cfg["norm"], bias, cfg["groups"][0], cfg["groups"][1], cfg["scale"])
    w0, i0, s0 = ref.moe_router(b, k, cfg["scoring"], cfg["norm"], bias, cfg["groups"][0], cfg["groups"][1], cfg["scale"])
    assert torch.equal(i1.sort(-1).values, i0.sort(-1).values)
    o1, o0 = i1.argsort(-1), i0.argsort(-1)
    assert torch.allclose(w1.gather(1, o1), w0.gather(1, o0), rtol=1e-5, atol=1e-6)
    assert torch.allclose(s1, s0, rtol=1e-5, atol=1e-7)
    assert torch.equal(i1._moe_hist.long(), torch.bincount(i0.reshape(-1), minlength=E))
    # gradients through the weights and through the scores (aux loss)
    gw, gs = torch.randn_like(w0), torch.randn_like(s0) * 0.1
    (w1.gather(1, o1) * gw).sum().add((s1 * gs).sum()).backward()
    (w0.gather(1, o0) * gw).sum().add((s0 * gs).sum()).backward()
    assert torch.allclose(a.grad, b.grad, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("R,G,N,K", [(1000, 8, 512, 256), (77, 16, 1536, 2048), (4096, 128, 1536, 2048), (5, 4, 64, 64)])
def test_grouped_gemm_ragged(R, G, N, K):
    from chatlearn_b200.ops import native
    torch.manual_seed(1)
    a = torch.randn(R, K, device=_dev()).bfloat16()
    b = (torch.randn(G, N, K, device=_dev()) * 0.05).bfloat16()
    cuts = torch.sort(torch.randint(0, R + 1, (G - 1,))).values.tolist()
    if G > 3:
        cuts[1] = cuts[0]                                   # an empty group
    bounds = [0] + cuts + [R]
    off = torch.tensor(bounds, dtype=torch.long, device=_dev())
    c = native.C.grouped_gemm_bf16_nt(a, b, off)
    want = torch.empty(R, N, device=_dev())
    for g in range(G):
        s, t = bounds[g], bounds[g + 1]
        want[s:t] = a[s:t].float() @ b[g].float().t()
    assert native.C.gemm_last_status() == 0
    err = (c.float() - want).norm() / want.norm()
    assert err < 5e-3, err


def test_moe_experts_forward_backward():
    from chatlearn_b200 import ops
    from chatlearn_b200.ops import reference as ref
    torch.manual_seed(2)
    T, H, F, E, k = 300, 256, 128, 16, 4
    dev = _dev()
    x = torch.randn(T, H, device=dev).bfloat16()
    w13 = (torch.randn(E, 2 * F, H, device=dev) * 0.05).bfloat16()
    w2 = (torch.randn(E, H, F, device=dev) * 0.05).bfloat16()
    logits = torch.randn(T, E, device=dev)
    wts, idx, _ = ref.moe_router(logits, k)
    args1 = [t.clone().requires_grad_(True) for t in (x, w13, w2, wts)]
    args0 = [t.float().clone().requires_grad_(True) for t in (x, w13, w2, wts)]
    y1 = ops.moe_experts(args1[0], args1[1], args1[2], args1[3], idx)
    y0 = ref.moe_experts(args0[0], args0[1], args0[2], args0[3], idx)
    assert (y1.float() - y0).norm() / y0.norm() < 2e-2
    g = torch.randn_like(y0)
    y1.backward(g.bfloat16())
    y0.backward(g)
    for a, b, name in zip(args1, args0, ("x", "w13", "w2", "weights")):
        rel = (a.grad.float() - b.grad).norm() / b.grad.norm()
        assert rel < 3e-2, (name, rel)
    assert ops.launch_counts["grouped_gemm_bf16_nt"] >= 2
