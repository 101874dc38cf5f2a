"""Numerics of the sm_100a kernels against plain PyTorch fp32 statements of the
same ops.  Needs a CUDA device (B200)."""
import math

import pytest
import torch

from chatlearn_b200 import ops
from chatlearn_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def native():
    from chatlearn_b200.ops import native as n
    return n


def _close(a, b, rtol, atol):
    a, b = a.float().cpu(), b.float().cpu()
    assert torch.allclose(a, b, rtol=rtol, atol=atol), f"max abs diff {(a - b).abs().max().item():.3e}"


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("shape", [(7, 256), (130, 4096), (0, 512)])
def test_rmsnorm(native, dtype, tol, shape):
    torch.manual_seed(0)
    x = torch.randn(*shape, device=DEV).to(dtype).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(shape[-1], device=DEV)).to(dtype).requires_grad_(True)
    y = native.rmsnorm(x, w, 1e-6)
    g = torch.randn_like(y)
    if shape[0]:
        y.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = ref.rmsnorm(xr, wr, 1e-6)
    _close(y, yr, tol, tol)
    if shape[0]:
        yr.backward(g.float())
        _close(x.grad, xr.grad, tol, tol)
        _close(w.grad, wr.grad, tol * 4, tol * shape[0] ** 0.5)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_swiglu(native, dtype, tol):
    torch.manual_seed(1)
    gu = torch.randn(33, 2 * 704, device=DEV).to(dtype).requires_grad_(True)
    y = native.swiglu(gu)
    g = torch.randn_like(y)
    y.backward(g)
    gr = gu.detach().float().requires_grad_(True)
    yr = ref.swiglu(gr)
    yr.backward(g.float())
    _close(y, yr, tol, tol)
    _close(gu.grad, gr.grad, tol, tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("d,with_norm", [(128, True), (64, True), (128, False)])
def test_qk_norm_rope(native, dtype, tol, d, with_norm):
    torch.manual_seed(2)
    T, nq, nkv = 37, 4, 2
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=DEV).to(dtype).requires_grad_(True)
    qw = (1 + 0.1 * torch.randn(d, device=DEV)).to(dtype).requires_grad_(with_norm)
    kw = (1 + 0.1 * torch.randn(d, device=DEV)).to(dtype).requires_grad_(with_norm)
    pos = torch.randint(0, 5000, (T,), device=DEV)

    def run(fn, qkv_, qw_, kw_):
        q = qkv_[:, :nq * d].view(T, nq, d)
        k = qkv_[:, nq * d:(nq + nkv) * d].view(T, nkv, d)
        return fn(q, k, qw_ if with_norm else None, kw_ if with_norm else None, 1e-6, pos, 1e6)

    q1, k1 = run(native.qk_norm_rope, qkv, qw, kw)
    gq, gk = torch.randn_like(q1), torch.randn_like(k1)
    (q1 * gq).sum().backward(retain_graph=True)
    (k1 * gk).sum().backward()
    qkv_r = qkv.detach().float().requires_grad_(True)
    qw_r, kw_r = qw.detach().float().requires_grad_(with_norm), kw.detach().float().requires_grad_(with_norm)
    q2, k2 = run(ref.qk_norm_rope, qkv_r, qw_r, kw_r)
    ((q2 * gq.float()).sum() + (k2 * gk.float()).sum()).backward()
    _close(q1, q2, tol, tol)
    _close(k1, k2, tol, tol)
    _close(qkv.grad[:, :(nq + nkv) * d], qkv_r.grad[:, :(nq + nkv) * d], tol, tol * 2)
    if with_norm:
        _close(qw.grad, qw_r.grad, tol * 4, tol * 8)
        _close(kw.grad, kw_r.grad, tol * 4, tol * 8)


def test_grpo_loss(native):
    torch.manual_seed(3)
    n = 5000
    lp = (-2 + torch.randn(n, device=DEV)).requires_grad_(True)
    old = lp.detach() + 0.3 * torch.randn(n, device=DEV)
    old[:50] -= 15.0            # exercise the diff clip
    refl = lp.detach() + 0.2 * torch.randn(n, device=DEV)
    adv = torch.randn(n, device=DEV) * 3
    mask = (torch.rand(n, device=DEV) > 0.3).float()
    ent = torch.rand(n, device=DEV).requires_grad_(True)
    kw = dict(pos_clip=0.2, neg_clip=0.2, diff_clip=10.0, final_clip=3.0, kl_coef=0.01, entropy_coef=0.02,
              inv_norm=1.0 / 1234)
    t1, s1 = native.grpo_loss_fused(lp, old, refl, adv, mask, ent, **kw)
    t1.backward()
    lp2, ent2 = lp.detach().clone().requires_grad_(True), ent.detach().clone().requires_grad_(True)
    t2, s2 = ref.grpo_loss_fused(lp2, old, refl, adv, mask, ent2, **kw)
    t2.backward()
    _close(t1, t2, 1e-4, 1e-5)
    _close(s1, s2, 1e-4, 1e-2)
    _close(lp.grad, lp2.grad, 1e-4, 1e-7)
    _close(ent.grad, ent2.grad, 1e-5, 1e-8)


def test_gspo_loss(native):
    """Group-sequence loss: every token of a packed sequence uses the sequence's mean log-ratio; value, statistics
    and the gradients against the PyTorch statements."""
    torch.manual_seed(31)
    lens = [700, 1, 1300, 64, 2935]
    n = sum(lens)
    seq_ids = torch.repeat_interleave(torch.arange(len(lens), device=DEV), torch.tensor(lens, device=DEV))
    lp = (-2 + torch.randn(n, device=DEV)).requires_grad_(True)
    old = lp.detach() + 0.02 * torch.randn(n, device=DEV)
    old[seq_ids == 3] -= 15.0                       # this sequence's mean exceeds the diff clip
    refl = lp.detach() + 0.2 * torch.randn(n, device=DEV)
    adv = torch.randn(len(lens), device=DEV)[seq_ids] * 3
    mask = (torch.rand(n, device=DEV) > 0.3).float()
    mask[seq_ids == 1] = 0.0                        # a sequence with no loss tokens at all
    ent = torch.rand(n, device=DEV).requires_grad_(True)
    kw = dict(pos_clip=3e-3, neg_clip=4e-3, diff_clip=10.0, final_clip=3.0, kl_coef=0.01, entropy_coef=0.02,
              inv_norm=1.0 / 777)
    t1, s1 = native.gspo_loss_fused(lp, old, refl, adv, mask, seq_ids, len(lens), ent, **kw)
    t1.backward()
    lp2, ent2 = lp.detach().clone().requires_grad_(True), ent.detach().clone().requires_grad_(True)
    t2, s2 = ref.gspo_loss_fused(lp2, old, refl, adv, mask, seq_ids, len(lens), ent2, **kw)
    t2.backward()
    _close(t1, t2, 1e-4, 1e-5)
    _close(s1, s2, 1e-4, 1e-2)
    _close(lp.grad, lp2.grad, 1e-4, 1e-7)
    _close(ent.grad, ent2.grad, 1e-5, 1e-8)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_adamw_and_sumsq(native, out_dtype):
    torch.manual_seed(4)
    n = 100003 * 4
    master = torch.randn(n, device=DEV)
    grad = torch.randn(n, device=DEV)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    out = torch.empty(n, device=DEV, dtype=out_dtype)
    ref_state = [t.clone() for t in (master, m, v)]
    out_r = torch.empty(n, device=DEV, dtype=out_dtype)
    scale = torch.tensor(0.5, device=DEV)
    for step in (1, 2, 3):
        native.adamw_step(master, grad, m, v, out, step, 1e-3, 0.9, 0.95, 1e-8, 0.01, scale)
        ref.adamw_step(ref_state[0], grad, ref_state[1], ref_state[2], out_r, step, 1e-3, 0.9, 0.95, 1e-8, 0.01, scale)
    _close(master, ref_state[0], 1e-5, 1e-6)
    _close(out, out_r, 1e-2 if out_dtype == torch.bfloat16 else 1e-5, 1e-6)
    _close(native.sumsq(grad), grad.double().pow(2).sum().float(), 1e-5, 0)
    _close(native.sumsq(grad.bfloat16()), grad.bfloat16().double().pow(2).sum().float(), 1e-5, 0)


@pytest.mark.parametrize("V", [1024, 151936])
def test_lmhead_logprob_cublas_path(native, V):
    torch.manual_seed(5)
    T, H = 300, 256
    native.set_gemm_impl("cublas")
    try:
        h = (torch.randn(T, H, device=DEV) * 0.5).bfloat16().requires_grad_(True)
        w = (torch.randn(V, H, device=DEV) * 0.05).bfloat16().requires_grad_(True)
        lab = torch.randint(0, V, (T,), device=DEV)
        lp, ent = native.lmhead_logprob_entropy(h, w, lab, 1.0, chunk=128)
        g1, g2 = torch.randn(T, device=DEV), 0.1 * torch.randn(T, device=DEV)
        (lp * g1 + ent * g2).sum().backward()
        hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
        z = hr @ wr.t()
        lpr = ref.logprobs_from_logits(z, lab)
        entr = ref.entropy_from_logits(z)
        (lpr * g1 + entr * g2).sum().backward()
        _close(lp, lpr, 2e-2, 2e-2)
        _close(ent, entr, 2e-2, 2e-2)
        # gradients pass through bf16 dlogits: compare in relative Frobenius norm
        for a, b in ((h.grad, hr.grad), (w.grad, wr.grad)):
            rel = (a.float() - b).norm() / b.norm()
            assert rel < 2e-2, rel
    finally:
        native.set_gemm_impl("tcgen05")


def test_sampler(native):
    torch.manual_seed(6)
    B, V = 64, 5000
    logits = torch.randn(B, V, device=DEV) * 3
    u = torch.rand(B, device=DEV)
    for kw in (dict(temperature=1.0), dict(temperature=0.7, top_k=20), dict(temperature=1.0, top_p=0.9),
               dict(temperature=0.8, top_k=50, top_p=0.95, min_p=0.01), dict(temperature=0.0)):
        ids, lp = native.sample(logits, u, **kw)
        ids_r, lp_r = ref.sample(logits, u, **kw)
        agree = (ids == ids_r).float().mean().item()
        assert agree >= 0.95, (kw, agree)       # fp32 summation order may move a boundary draw
        same = ids == ids_r
        _close(lp[same], lp_r[same], 1e-4, 1e-4)
    # distribution check: empirical frequencies follow softmax
    z = torch.tensor([[2.0, 1.0, 0.0, -1.0]], device=DEV).repeat(20000, 1)
    ids, _ = native.sample(z, torch.rand(20000, device=DEV), temperature=1.0)
    freq = torch.bincount(ids, minlength=4).float() / 20000
    _close(freq, torch.softmax(z[0], -1), 0.05, 0.01)


def test_penalties(native):
    torch.manual_seed(7)
    z = torch.randn(4, 100, device=DEV)
    counts = torch.randint(0, 3, (4, 100), device=DEV, dtype=torch.int32)
    pm = torch.rand(4, 100, device=DEV) > 0.8
    a = native.apply_penalties(z, counts, 0.5, 0.2, 1.3, pm)
    b = ref.apply_penalties(z, counts, 0.5, 0.2, 1.3, pm)
    _close(a, b, 1e-6, 1e-6)


@pytest.mark.parametrize("d,nq,nkv,bs", [(128, 8, 2, 64), (64, 4, 4, 16), (128, 32, 8, 64)])
def test_paged_attention_decode(native, d, nq, nkv, bs):
    torch.manual_seed(8)
    B, nb = 5, 64
    seq_lens = torch.tensor([1, 63, 64, 200, 517][:B], dtype=torch.int32, device=DEV)
    maxb = int((seq_lens.max().item() + bs - 1) // bs)
    kc = torch.randn(nb * 4, bs, nkv, d, device=DEV).bfloat16()
    vc = torch.randn(nb * 4, bs, nkv, d, device=DEV).bfloat16()
    perm = torch.randperm(nb * 4, device=DEV)[:B * maxb].view(B, maxb).int()
    q = torch.randn(B, nq, d, device=DEV).bfloat16()
    o_r = ref.paged_attention(q, kc, vc, perm, seq_lens, None, None)
    for impl in ("tc", "simt"):          # tensor-core kernel (64-token blocks) and the SIMT kernel
        native.set_decode_impl(impl)
        o = native.paged_attention(q, kc, vc, perm, seq_lens, None, None)
        _close(o, o_r, 2e-2, 2e-2)
    native.set_decode_impl("tc")
    # long context: exercises the split-KV path and its merge kernel
    if bs == 64:
        sl2 = torch.tensor([4000], dtype=torch.int32, device=DEV)
        nb2 = (4000 + bs - 1) // bs
        bt2 = torch.randperm(nb * 4, device=DEV)[:nb2].view(1, nb2).int()
        q1 = torch.randn(1, nq, d, device=DEV).bfloat16()
        _close(native.paged_attention(q1, kc, vc, bt2, sl2, None, None),
               ref.paged_attention(q1, kc, vc, bt2, sl2, None, None), 2e-2, 2e-2)
    # chunk continuation: 3 query tokens for the longest sequence, 1 for the others
    q_lens = torch.tensor([1, 1, 1, 1, 3][:B], dtype=torch.int32, device=DEV)
    q2 = torch.randn(int(q_lens.sum()), nq, d, device=DEV).bfloat16()
    o2 = native.paged_attention(q2, kc, vc, perm, seq_lens, q_lens, None)
    o2_r = ref.paged_attention(q2, kc, vc, perm, seq_lens, q_lens, None)
    _close(o2, o2_r, 2e-2, 2e-2)


def test_kv_append(native):
    k = torch.randn(10, 2, 64, device=DEV).bfloat16()
    v = torch.randn(10, 2, 64, device=DEV).bfloat16()
    kc, vc = torch.zeros(4, 8, 2, 64, device=DEV).bfloat16(), torch.zeros(4, 8, 2, 64, device=DEV).bfloat16()
    kc2, vc2 = kc.clone(), vc.clone()
    slots = torch.tensor([3, 9, 31, 0, -1, 17, 18, 19, 20, 8], device=DEV)
    native.kv_append(k, v, kc, vc, slots)
    ref.kv_append(k, v, kc2, vc2, slots)
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)


def test_weight_sync_kernel_local(native):
    """Descriptor-table kernel against the planner's gather-then-slice oracle (one GPU:
    FSDP-layout fp32 source -> TP=2 rollout layout bf16, both 'ranks' emulated as buffers)."""
    from chatlearn_b200.models.nn import CausalLM, PRESETS
    from chatlearn_b200.synchronizer.kernel_executor import KernelExecutor
    from chatlearn_b200.synchronizer.parameter_sync import layout_of_model
    from chatlearn_b200.synchronizer.plan import build_plan, validate_plan
    arch = PRESETS["tiny_qwen3"]()
    src = CausalLM(arch, dtype=torch.float32, device=DEV).init_weights(3)
    full = src.hf_state_dict()
    for tp_rank in range(2):
        dst = CausalLM(arch, dtype=torch.bfloat16, device=DEV, tp=2, tp_rank=tp_rank)
        want = CausalLM(arch, dtype=torch.bfloat16, device=DEV, tp=2, tp_rank=tp_rank)
        want.load_hf_state_dict(full)
        plan = build_plan([layout_of_model(src, 0, prefix="s/")], [layout_of_model(dst, 0, prefix="d/")])
        validate_plan(plan, [layout_of_model(dst, 0, prefix="d/")])
        ex = KernelExecutor(plan, 0, 1)
        ex.run({f"s/{b.name}": b.flat for b in src.blocks}, {f"d/{b.name}": b.flat for b in dst.blocks})
        torch.cuda.synchronize()
        for a, b in zip(dst.blocks, want.blocks):
            assert torch.equal(a.flat, b.flat), a.name


@pytest.mark.parametrize("with_norm", [True, False])
def test_qkv_rope_append_matches_the_separate_kernels(native, with_norm):
    """q/k norm + RoPE + cache append in one launch against the three statements it replaces."""
    torch.manual_seed(41)
    T, nq, nkv, D, bs, nb = 37, 8, 2, 128, 16, 12
    qkv = torch.randn(T, (nq + 2 * nkv) * D, device=DEV).bfloat16()
    qw = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16() if with_norm else None
    kw = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16() if with_norm else None
    pos = torch.randint(0, 4000, (T,), device=DEV)
    slots = torch.randperm(nb * bs, device=DEV)[:T]
    slots[5] = -1                                            # a row whose cache writes are skipped
    caches = [[torch.zeros(nb, bs, nkv, D, device=DEV, dtype=torch.bfloat16) for _ in range(2)] for _ in range(2)]
    q1 = native.qkv_rope_append(qkv, nq, nkv, D, qw, kw, 1e-6, pos, 1e6, slots, caches[0][0], caches[0][1])
    keep = slots >= 0
    q2 = ref.qkv_rope_append(qkv[keep], nq, nkv, D, qw, kw, 1e-6, pos[keep], 1e6, slots[keep], caches[1][0], caches[1][1])
    _close(q1[keep], q2, 2e-2, 2e-2)
    _close(caches[0][0], caches[1][0], 2e-2, 2e-2)
    assert torch.equal(caches[0][1], caches[1][1])


def test_grouped_decode_attention_matches_the_per_sequence_kernel(native):
    """Sequences whose block tables start with the same blocks: the shared blocks attended once per group plus the
    per-sequence remainder, merged by log-sum-exp, must equal the per-sequence kernel over the whole context."""
    import math
    torch.manual_seed(51)
    nq, nkv, d, bs = 8, 2, 128, 64
    groups = [(5, 4, [70, 1, 130, 64, 200]), (3, 8, [10, 500, 65, 3, 90, 64, 1, 129]), (2, 0, [300, 77])]   # (shared blocks, -, suffix tokens)
    singles = [100, 640]
    tables, ctx, members = [], [], []
    nb_total = 0
    for shared, _, tails in groups:
        base = list(range(nb_total, nb_total + shared))
        nb_total += shared
        rows = []
        for tail in tails:
            own = math.ceil(tail / bs)
            tables.append(base + list(range(nb_total, nb_total + own)))
            nb_total += own
            ctx.append(shared * bs + tail)
            rows.append(len(tables) - 1)
        members.append((rows, shared))
    for n in singles:
        own = math.ceil(n / bs)
        tables.append(list(range(nb_total, nb_total + own)))
        nb_total += own
        ctx.append(n)
    B, width = len(tables), max(len(t) for t in tables)
    bt = torch.zeros(B, width, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t)
    perm = torch.randperm(nb_total + 3).int()                      # physical block ids in no particular order
    bt = perm[bt.long()].to(DEV)
    kc = torch.randn(nb_total + 3, bs, nkv, d, device=DEV).bfloat16()
    vc = torch.randn(nb_total + 3, bs, nkv, d, device=DEV).bfloat16()
    q = torch.randn(B, nq, d, device=DEV).bfloat16()
    sl = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    G = 6
    grp_q = torch.full((G, 8), -1, dtype=torch.int32)
    grp_nblk = torch.zeros(G, dtype=torch.int32)
    blk_start = torch.zeros(B, dtype=torch.int32)
    g = 1                                                          # leave group slot 0 unused on purpose
    for rows, shared in members:
        if shared == 0:
            continue
        grp_q[g, :len(rows)] = torch.tensor(rows, dtype=torch.int32)
        grp_nblk[g] = shared
        blk_start[rows] = shared
        g += 1
    scale = 1 / math.sqrt(d)
    want = native.C.paged_decode_tc(q, kc, vc, bt, None, sl, scale, 1)
    for np_, ns_ in ((1, 1), (2, 1), (3, 2)):
        got = native.C.paged_decode_tc_grouped(q, kc, vc, bt, sl, grp_q.to(DEV), grp_nblk.to(DEV), blk_start.to(DEV), scale, np_, ns_)
        _close(got, want, 2e-2, 2e-2)
    ref_out = ref.paged_attention(q, kc, vc, bt, sl, None, scale)
    _close(want, ref_out, 2e-2, 2e-2)


@pytest.mark.parametrize("heads,splits", [(16, 1), (16, 3), (40, 0), (5, 2)])
def test_mla_paged_decode_matches_fp32_statements(heads, splits):
    """Latent-attention decode kernel (latent 512 + rotary 64) against fp32 statements over the same paged cache:
    ragged lengths (one below a block, one at a block edge), head counts that are not a multiple of the 16-row tile,
    one CTA per sequence and several splits of the context."""
    from chatlearn_b200.models.nn.mla import latent_paged_attention
    from chatlearn_b200.ops import native
    torch.manual_seed(3)
    dev = "cuda"
    lens = [1, 63, 64, 65, 700, 1531, 128, 2049]
    B, bs, D, lora = len(lens), 64, 576, 512
    max_blocks = (max(lens) + bs - 1) // bs + 1
    nblocks = sum((n + bs - 1) // bs for n in lens) + 4
    cache = (torch.randn(nblocks, bs, 1, D, device=dev) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(nblocks, device=dev).to(torch.int32)
    bt = torch.zeros(B, max_blocks, dtype=torch.int32, device=dev)
    at = 0
    for i, n in enumerate(lens):
        k = (n + bs - 1) // bs
        bt[i, :k] = perm[at:at + k]
        at += k
    q = (torch.randn(B, heads, D, device=dev) * 0.3).to(torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    scale = 192 ** -0.5
    out = native.C.mla_paged_decode(q, cache, bt, sl, scale, splits)
    ref = latent_paged_attention(q.float(), cache.float(), lora, bt, sl, None, 1, scale)
    assert out.shape == (B, heads, lora) and out.dtype == torch.bfloat16
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2, err
    # through the op table (automatic split choice)
    from chatlearn_b200 import ops
    out2 = ops.mla_paged_decode(q, cache, lora, bt, sl, scale)
    assert (out2.float() - ref).abs().max().item() < 2e-2
