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


@pytest.mark.parametrize("G,K,N,M", [(8, 256, 192, 320), (40, 128, 512, 64)])
def test_grouped_gemm_backward_layouts(G, K, N, M):
    """Input-gradient (NN) and weight-gradient (ragged contraction) forms of the grouped GEMM against fp32
    statements: groups padded to 64 rows with zero rows in between, some groups empty."""
    from chatlearn_b200.ops import native
    torch.manual_seed(5)
    dev = _dev()
    counts = torch.randint(0, 150, (G,))
    counts[1] = 0
    counts[G - 1] = 0
    padded = (counts + 63) // 64 * 64
    off = torch.zeros(G + 1, dtype=torch.long)
    off[1:] = padded.cumsum(0)
    R = int(off[-1]) + 64                                    # a tail no group covers
    a = torch.zeros(R, K)
    bt = torch.zeros(R, N)
    for g in range(G):
        s, n = int(off[g]), int(counts[g])
        a[s:s + n] = torch.randn(n, K)
        bt[s:s + n] = torch.randn(n, N)
    a, bt = a.to(dev).bfloat16(), bt.to(dev).bfloat16()
    offd = off.to(dev)
    # NN: c[r] = a[r] @ w[g], w [G, K, N]
    w = (torch.randn(G, K, N, device=dev) * 0.1).bfloat16()
    c = native.C.grouped_gemm_bf16_nn(a, w, offd)
    for g in range(G):
        s, t = int(off[g]), int(off[g + 1])
        if t > s:
            want = a[s:t].float() @ w[g].float()
            assert (c[s:t].float() - want).norm() <= 5e-3 * max(want.norm().item(), 1e-6), g
    # TN: out[g] = a[rows of g]^T @ bt[rows of g], a as [R, M = K]
    out = torch.full((G, K, N), 7.0, device=dev).bfloat16()
    native.C.grouped_gemm_bf16_tn(a, bt, offd, out, False)
    acc = torch.ones(G, K, N, device=dev)
    native.C.grouped_gemm_bf16_tn(a, bt, offd, acc, True)
    assert native.C.gemm_last_status() == 0
    for g in range(G):
        s, t = int(off[g]), int(off[g + 1])
        want = a[s:t].float().t() @ bt[s:t].float()
        tol = 5e-3 * max(want.norm().item(), 1.0)
        assert (out[g].float() - want).norm() <= tol, g
        assert (acc[g] - 1.0 - want).norm() <= 1e-3 * max(want.norm().item(), 1.0), g
    # second shape family: M (rows of the weight) not a multiple of the 128-row tile
    a2 = torch.zeros(R, M)
    for g in range(G):
        s, n = int(off[g]), int(counts[g])
        a2[s:s + n] = torch.randn(n, M)
    a2 = a2.to(dev).bfloat16()
    out2 = torch.empty(G, M, N, device=dev, dtype=torch.bfloat16)
    native.C.grouped_gemm_bf16_tn(a2, bt, offd, out2, False)
    for g in range(G):
        s, t = int(off[g]), int(off[g + 1])
        want = a2[s:t].float().t() @ bt[s:t].float()
        assert (out2[g].float() - want).norm() <= 5e-3 * max(want.norm().item(), 1.0), g


def test_moe_experts_backward_uses_the_grouped_kernels_with_empty_experts():
    from chatlearn_b200 import ops
    from chatlearn_b200.ops import reference as ref
    torch.manual_seed(4)
    T, H, F, E, k = 90, 192, 96, 64, 2                        # 180 pairs over 64 experts: several experts get no token
    dev = _dev()
    x = torch.randn(T, H, device=dev).bfloat16()
    w13 = (torch.randn(E, 2 * F, H, device=dev) * 0.05).bfloat16()
    w2 = (torch.randn(E, H, F, device=dev) * 0.05).bfloat16()
    wts, idx, _ = ref.moe_router(torch.randn(T, E, device=dev), k)
    assert torch.bincount(idx.reshape(-1), minlength=E).min().item() == 0
    args1 = [t.clone().requires_grad_(True) for t in (x, w13, w2, wts)]
    args0 = [t.float().clone().requires_grad_(True) for t in (x, w13, w2, wts)]
    before = ops.launch_counts["grouped_gemm_bf16_tn"], ops.library_counts["grouped_gemm_bwd"]
    y1 = ops.moe_experts(args1[0], args1[1], args1[2], args1[3], idx)
    y0 = ref.moe_experts(args0[0], args0[1], args0[2], args0[3], idx)
    assert (y1.float() - y0).norm() / y0.norm() < 2e-2
    g = torch.randn_like(y0)
    y1.backward(g.bfloat16())
    y0.backward(g)
    for a, b, name in zip(args1, args0, ("x", "w13", "w2", "weights")):
        rel = (a.grad.float() - b.grad).norm() / b.grad.norm()
        assert rel < 3e-2, (name, rel)
    assert ops.launch_counts["grouped_gemm_bf16_tn"] == before[0] + 2
    assert ops.library_counts["grouped_gemm_bwd"] == before[1]
    # without a tape the rows are packed densely (no padding)
    with torch.no_grad():
        y2 = ops.moe_experts(x, w13, w2, wts, idx)
    assert (y2.float() - y0.detach()).norm() / y0.norm() < 2e-2


def test_grouped_mlp_with_host_counts_trains_on_the_grouped_kernels():
    """Rows packed densely by expert with the group sizes on the host (what the expert-parallel exchange delivers):
    with a tape they are moved into the padded layout, so the backward takes the grouped kernels."""
    from chatlearn_b200 import ops
    from chatlearn_b200.ops import reference as ref
    torch.manual_seed(8)
    E, H, F = 6, 128, 64
    counts = [70, 0, 128, 5, 64, 33]
    dev = _dev()
    R = sum(counts)
    xs = torch.randn(R, H, device=dev).bfloat16()
    w13 = (torch.randn(E, 2 * F, H, device=dev) * 0.05).bfloat16()
    w2 = (torch.randn(E, H, F, device=dev) * 0.05).bfloat16()
    a1 = [t.clone().requires_grad_(True) for t in (xs, w13, w2)]
    a0 = [t.float().clone().requires_grad_(True) for t in (xs, w13, w2)]
    before = ops.launch_counts["grouped_gemm_bf16_tn"], ops.library_counts["grouped_gemm_bwd"]
    y1 = ops.grouped_mlp(a1[0], a1[1], a1[2], counts)
    y0 = ref.grouped_mlp(a0[0], a0[1], a0[2], counts)
    assert y1.shape == y0.shape and (y1.float() - y0).norm() / y0.norm() < 2e-2
    g = torch.randn_like(y0)
    y1.backward(g.bfloat16())
    y0.backward(g)
    for a, b, name in zip(a1, a0, ("x", "w13", "w2")):
        rel = (a.grad.float() - b.grad).norm() / b.grad.norm()
        assert rel < 3e-2, (name, rel)
    assert ops.launch_counts["grouped_gemm_bf16_tn"] == before[0] + 2 and ops.library_counts["grouped_gemm_bwd"] == before[1]
