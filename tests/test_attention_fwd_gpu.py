"""Packed causal attention forward kernel against fp32 SDPA per segment."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, cu, scale, causal=True):
    outs = []
    rep = q.shape[1] // k.shape[1]
    for s, e in zip(cu[:-1], cu[1:]):
        if e == s:
            continue
        qs = q[s:e].float().transpose(0, 1).unsqueeze(0)
        ks = k[s:e].float().transpose(0, 1).unsqueeze(0).repeat_interleave(rep, 1)
        vs = v[s:e].float().transpose(0, 1).unsqueeze(0).repeat_interleave(rep, 1)
        o = torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=causal, scale=scale)
        outs.append(o.squeeze(0).transpose(0, 1))
    return torch.cat(outs, 0)


@pytest.mark.parametrize("nq,nkv,D", [(32, 8, 128), (4, 2, 64), (8, 8, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_varlen_forward_matches_sdpa(nq, nkv, D, causal):
    from chatlearn_b200 import ops
    from chatlearn_b200.ops import native
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    lens = [1, 63, 64, 65, 200, 0, 1000, 129]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    qkv = torch.randn(T, (nq + 2 * nkv) * D, device=dev).bfloat16()
    q = qkv[:, :nq * D].view(T, nq, D)                       # strided rows, as sliced from a fused projection
    k = qkv[:, nq * D:(nq + nkv) * D].view(T, nkv, D)
    v = qkv[:, (nq + nkv) * D:].view(T, nkv, D)
    scale = 1.0 / math.sqrt(D)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    with torch.no_grad():
        if causal:
            before = ops.launch_counts["attn_varlen_fwd"]
            out = ops.attention_varlen(q, k, v, cu_t, max(lens), scale)
            assert ops.launch_counts["attn_varlen_fwd"] == before + 1
        else:
            out, _ = native.C.attn_varlen_fwd(q, k, v, cu_t, scale, False)
    want = _ref(q, k, v, cu, scale, causal)
    err = (out.float() - want).abs().max().item()
    assert err < 2e-2, err
    # log-sum-exp of a row: check against the definition on one segment
    out2, lse = native.C.attn_varlen_fwd(q, k, v, cu_t, scale, True)
    s, e = cu[4], cu[5]
    logits = torch.einsum("qd,kd->qk", q[s:e, 0].float(), k[s:e, 0].float()) * scale
    logits = logits.masked_fill(torch.triu(torch.ones(e - s, e - s, device=dev, dtype=torch.bool), 1), float("-inf"))
    assert torch.allclose(lse[0, s:e], torch.logsumexp(logits, -1), rtol=1e-3, atol=1e-2)


def test_gradient_pass_at_head_dim_64_uses_library_and_matches():
    from chatlearn_b200 import ops
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    q = torch.randn(300, 8, 64, device=dev).bfloat16().requires_grad_(True)
    k = torch.randn(300, 2, 64, device=dev).bfloat16()
    v = torch.randn(300, 2, 64, device=dev).bfloat16()
    cu = torch.tensor([0, 100, 300], dtype=torch.int32, device=dev)
    before = ops.launch_counts["attn_varlen_fwd"]
    o = ops.attention_varlen(q, k, v, cu, 200, None)
    assert ops.launch_counts["attn_varlen_fwd"] == before          # no backward kernel for head dim 64: the library runs
    with torch.no_grad():
        o2 = ops.attention_varlen(q.detach(), k, v, cu, 200, None)
    assert (o.float() - o2.float()).abs().max() < 2e-2


@pytest.mark.parametrize("nq,nkv", [(8, 2), (4, 4)])
@pytest.mark.parametrize("causal", [True, False])
def test_tcgen05_forward_matches_sdpa(nq, nkv, causal):
    """The tensor-memory kernel (head dim 128) on ragged lengths: single rows, lengths around the 64-key block
    and the 128-row tile, an empty sequence, and sequences long enough for many key blocks."""
    from chatlearn_b200.ops import native
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    D = 128
    lens = [1, 63, 64, 65, 127, 128, 129, 200, 0, 1000, 2730, 5]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    qkv = torch.randn(T, (nq + 2 * nkv) * D, device=dev).bfloat16()
    q = qkv[:, :nq * D].view(T, nq, D)
    k = qkv[:, nq * D:(nq + nkv) * D].view(T, nkv, D)
    v = qkv[:, (nq + nkv) * D:].view(T, nkv, D)
    scale = 1.0 / math.sqrt(D)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    out, lse = native.C.attn_fwd_sm100(q, k, v, cu_t, scale, causal)
    torch.cuda.synchronize()
    assert native.C.attn_sm100_last_status() == 0, "a bounded wait inside the attention kernel ran out"
    want = _ref(q, k, v, cu, scale, causal)
    err = (out.float() - want).abs().max().item()
    assert err < 2e-2, err
    for si in (3, 9, 10):
        s, e = cu[si], cu[si + 1]
        logits = torch.einsum("qd,kd->qk", q[s:e, 1].float(), k[s:e, 1 * nkv // nq].float()) * scale
        if causal:
            logits = logits.masked_fill(torch.triu(torch.ones(e - s, e - s, device=dev, dtype=torch.bool), 1), float("-inf"))
        assert torch.allclose(lse[1, s:e], torch.logsumexp(logits, -1), rtol=1e-3, atol=1e-2)


def test_tcgen05_forward_large_scores_exercise_the_lazy_rescale():
    """Scores that grow along the sequence force the running maximum far past the reference maximum, so the
    accumulator in tensor memory is rescaled many times."""
    from chatlearn_b200.ops import native
    dev = torch.device("cuda", 0)
    torch.manual_seed(4)
    T, nq, nkv, D = 1500, 4, 2, 128
    q = torch.randn(T, nq, D, device=dev).bfloat16()
    ramp = torch.linspace(0.2, 6.0, T, device=dev).view(T, 1, 1)
    k = (torch.randn(T, nkv, D, device=dev) * ramp).bfloat16()
    v = torch.randn(T, nkv, D, device=dev).bfloat16()
    cu = [0, 700, 1500]
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    scale = 1.0 / math.sqrt(D)
    out, _ = native.C.attn_fwd_sm100(q, k, v, cu_t, scale, True)
    torch.cuda.synchronize()
    assert native.C.attn_sm100_last_status() == 0
    want = _ref(q, k, v, cu, scale, True)
    assert (out.float() - want).abs().max().item() < 3e-2


def _ref_grads(q, k, v, cu, scale, causal, d_out):
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    _ref(qf, kf, vf, cu, scale, causal).backward(d_out.float())
    return qf.grad, kf.grad, vf.grad


@pytest.mark.parametrize("nq,nkv", [(8, 2), (4, 4)])
@pytest.mark.parametrize("causal", [True, False])
def test_tcgen05_backward_matches_fp32_sdpa(nq, nkv, causal):
    """dQ, dK, dV of the tensor-memory backward kernel against autograd through fp32 SDPA: ragged lengths,
    single-row sequences, an empty sequence, lengths around the 64-row query block and the 128-key block."""
    from chatlearn_b200 import ops
    from chatlearn_b200.ops import native
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    D = 128
    lens = [1, 63, 64, 65, 127, 128, 129, 200, 0, 700, 1, 1300]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    qkv = torch.randn(T, (nq + 2 * nkv) * D, device=dev).bfloat16().requires_grad_(True)
    q = qkv[:, :nq * D].view(T, nq, D)
    k = qkv[:, nq * D:(nq + nkv) * D].view(T, nkv, D)
    v = qkv[:, (nq + nkv) * D:].view(T, nkv, D)
    scale = 1.0 / math.sqrt(D)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    d_out = torch.randn(T, nq, D, device=dev).bfloat16()
    lib_before = ops.library_counts["attention_varlen"]
    if causal:
        out = ops.attention_varlen(q, k, v, cu_t, max(lens), scale)
        assert ops.library_counts["attention_varlen"] == lib_before, "the differentiable pass must run on the kernel"
    else:
        from chatlearn_b200.ops.native_attn import _AttnVarlen128
        out = _AttnVarlen128.apply(q, k, v, cu_t, scale, False)
    out.backward(d_out)
    torch.cuda.synchronize()
    assert native.C.attn_sm100_last_status() == 0 and native.C.attn_bwd_sm100_last_status() == 0
    g = qkv.grad.float()
    dq, dk, dv = g[:, :nq * D].view(T, nq, D), g[:, nq * D:(nq + nkv) * D].view(T, nkv, D), g[:, (nq + nkv) * D:].view(T, nkv, D)
    rq, rk, rv = _ref_grads(q, k, v, cu, scale, causal, d_out)
    for name, got, want in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        err = (got - want).abs().max().item()
        ref_mag = want.abs().max().item()
        assert err < 2e-2 * max(ref_mag, 1.0), (name, err, ref_mag)
