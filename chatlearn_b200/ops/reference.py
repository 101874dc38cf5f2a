"""Plain-PyTorch statements of every hot op.

These are (a) the CPU path of the framework (gloo plumbing runs, unit tests),
(b) the fp32 oracles the CUDA kernels are tested against and (c) the "library"
baseline mode on a GPU (torch matmul / SDPA), which is what the hand-written
sm_100a kernels are measured against.  Every function here is differentiable by
autograd unless it says otherwise.
"""
import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ norms / act
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype)


@torch.no_grad()
def add_rmsnorm_(resid: torch.Tensor, delta: torch.Tensor, w, eps: float):
    """In place ``resid += delta``; returns ``rmsnorm(resid) * w`` (``None`` when ``w`` is ``None``).
    Inference only: the residual stream is updated in place."""
    resid.add_(delta)
    return rmsnorm(resid, w, eps) if w is not None else None


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``[..., 2F] -> [..., F]``: silu(first half) * second half."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return F.linear(x, w, bias)


# ------------------------------------------------------------------ rope
def rope_cos_sin(positions: torch.Tensor, rot_dim: int, theta: float,
                 dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, device=positions.device,
                                        dtype=torch.float32) / rot_dim))
    ang = positions.float()[:, None] * inv[None, :]
    return ang.cos().to(dtype), ang.sin().to(dtype)


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float,
         rot_dim: Optional[int] = None) -> torch.Tensor:
    """Rotate-half (NeoX / HuggingFace) rotary embedding on ``x [T, heads, d]``;
    only the first ``rot_dim`` channels rotate."""
    d = x.shape[-1]
    rot_dim = rot_dim or d
    cos, sin = rope_cos_sin(positions, rot_dim, theta)
    xr = x[..., :rot_dim].float()
    x1, x2 = xr[..., : rot_dim // 2], xr[..., rot_dim // 2:]
    c, s = cos[:, None, :], sin[:, None, :]
    out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)
    if rot_dim < d:
        out = torch.cat([out, x[..., rot_dim:]], dim=-1)
    return out


def rope_mrope(x: torch.Tensor, positions3: torch.Tensor, theta: float, sections, interleaved: bool = False) -> torch.Tensor:
    """Multimodal rotary embedding (Qwen2-VL "mrope") on ``x [T, heads, d]``: frequency ``f`` of the
    ``d/2`` rotary frequencies takes its angle from the time, row or column position according to
    the section it falls in (``sections`` = three sizes summing to ``d/2``); ``positions3 [3, T]``.
    ``interleaved`` (Qwen3-VL): row and column frequencies are every third one (offsets 1 and 2) up to
    three times their section size, everything else is time."""
    d = x.shape[-1]
    half = d // 2
    assert sum(sections) == half, "mrope sections must sum to head_dim / 2"
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32, device=x.device) / d))
    if interleaved:
        f = torch.arange(half, device=x.device)
        comp = torch.zeros(half, dtype=torch.long, device=x.device)
        comp[(f % 3 == 1) & (f < 3 * sections[1])] = 1
        comp[(f % 3 == 2) & (f < 3 * sections[2])] = 2
    else:
        comp = torch.repeat_interleave(torch.arange(3, device=x.device), torch.tensor(list(sections), device=x.device))
    pos = positions3.to(torch.float32)[comp]                     # [d/2, T]: the position each frequency uses
    ang = (pos * inv[:, None]).t()                               # [T, d/2]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def qk_norm_rope(q, k, qw, kw, eps, positions, theta):
    """Per-head RMSNorm on q and k (Qwen3) followed by rotary embedding."""
    if qw is not None:
        q = rmsnorm(q, qw, eps)
        k = rmsnorm(k, kw, eps)
    return rope(q, positions, theta), rope(k, positions, theta)


# ------------------------------------------------------------------ attention
_VARLEN_LIB = {"probed": False, "fn": None}


def _library_varlen(q, k, v, cu_seqlens, max_seqlen, scale):
    """Library varlen attention for the GPU baseline mode (flash-attn if it runs on
    this GPU); ``None`` when no library kernel is usable."""
    st = _VARLEN_LIB
    if not st["probed"]:
        st["probed"] = True
        try:
            from flash_attn import flash_attn_varlen_func

            def fn(q, k, v, cu, mx, scale):
                return flash_attn_varlen_func(q, k, v, cu, cu, mx, mx, softmax_scale=scale, causal=True)
            # smoke call: a wheel without kernels for this architecture raises here
            t = torch.zeros(2, 1, 64, dtype=q.dtype, device=q.device)
            fn(t, t, t, torch.tensor([0, 2], dtype=torch.int32, device=q.device), 2, 0.125)
            st["fn"] = fn
        except Exception:
            st["fn"] = None
    if st["fn"] is None:
        return None
    if max_seqlen is None or max_seqlen <= 0:
        max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item())
    return st["fn"](q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens.to(torch.int32), int(max_seqlen), scale)


def qkv_rope_append(qkv, nq, nkv, D, q_weight, k_weight, eps, positions, theta, slot_mapping, k_cache, v_cache):
    """Inference with a paged cache: split the packed ``qkv [T, (nq + 2 nkv) D]`` rows, apply the per-head RMSNorm
    (when weights are given) and RoPE to queries and keys, store keys and values into their cache slots and return
    the queries ``[T, nq, D]``."""
    T = qkv.shape[0]
    q = qkv[:, :nq * D].view(T, nq, D)
    k = qkv[:, nq * D:(nq + nkv) * D].view(T, nkv, D)
    v = qkv[:, (nq + nkv) * D:].view(T, nkv, D)
    q, k = qk_norm_rope(q, k, q_weight, k_weight, eps, positions, theta)
    kv_append(k, v, k_cache, v_cache, slot_mapping)
    return q


def attention_varlen(q, k, v, cu_seqlens, max_seqlen=None, scale=None, causal=True):
    """Packed (varlen) attention.  ``q [T,nq,dq]``, ``k [T,nkv,dq]``,
    ``v [T,nkv,dv]``, ``cu_seqlens [B+1]``; segments attend only to themselves."""
    T, nq, dq = q.shape
    nkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(dq)
    if q.is_cuda and causal and q.dtype in (torch.bfloat16, torch.float16) and v.shape[-1] == dq:
        out = _library_varlen(q, k, v, cu_seqlens, max_seqlen, scale)
        if out is not None:
            return out
    rep = nq // nkv
    cu = cu_seqlens.tolist()
    outs = []
    for s, e in zip(cu[:-1], cu[1:]):
        if e == s:
            continue
        qs = q[s:e].transpose(0, 1).unsqueeze(0)
        ks = k[s:e].transpose(0, 1).unsqueeze(0)
        vs = v[s:e].transpose(0, 1).unsqueeze(0)
        if rep > 1:
            ks = ks.repeat_interleave(rep, dim=1)
            vs = vs.repeat_interleave(rep, dim=1)
        o = F.scaled_dot_product_attention(qs, ks, vs, is_causal=causal, scale=scale)
        outs.append(o.squeeze(0).transpose(0, 1))
    return torch.cat(outs, dim=0) if outs else q.new_zeros(0, nq, v.shape[-1])


def attention_segments(q, k, v, q_starts, q_lens, k_starts, k_lens, scale=None, max_q=0, max_k=0):
    """Attention over explicit (query rows, key rows) segment pairs with a causal
    mask aligned bottom-right: the last query of a segment sees all of its keys.
    Segments of ``k`` may overlap (context-parallel prefixes)."""
    nq, nkv = q.shape[1], k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    rep = nq // nkv
    out = q.new_zeros(q.shape[0], nq, v.shape[-1])
    pieces = []
    for qs, ql, ks, kl in zip(q_starts.tolist(), q_lens.tolist(), k_starts.tolist(), k_lens.tolist()):
        if ql == 0:
            continue
        qq, kk, vv = q[qs:qs + ql].float(), k[ks:ks + kl].float(), v[ks:ks + kl].float()
        if rep > 1:
            kk, vv = kk.repeat_interleave(rep, 1), vv.repeat_interleave(rep, 1)
        att = torch.einsum("qhd,khd->hqk", qq, kk) * scale
        qpos = torch.arange(kl - ql, kl, device=q.device)[:, None]
        kpos = torch.arange(kl, device=q.device)[None, :]
        att = att.masked_fill((kpos > qpos)[None], float("-inf"))
        o = torch.einsum("hqk,khd->qhd", att.softmax(-1), vv).to(q.dtype)
        pieces.append((qs, ql, o))
    if not pieces:
        return out
    # assemble without in-place writes on a leaf so autograd stays simple
    idx = torch.cat([torch.arange(qs, qs + ql, device=q.device) for qs, ql, _ in pieces])
    return out.index_copy(0, idx, torch.cat([o for _, _, o in pieces], 0))


def kv_append(k, v, k_cache, v_cache, slot_mapping):
    """Write ``k,v [T,nkv,d]`` into the paged caches ``[num_blocks, block, nkv, d]``
    at flat slots ``slot_mapping [T]`` (negative slot = skip)."""
    nb, bs = k_cache.shape[:2]
    ok = slot_mapping >= 0
    slots = slot_mapping[ok]
    k_cache.view(nb * bs, *k_cache.shape[2:])[slots] = k[ok].to(k_cache.dtype)
    v_cache.view(nb * bs, *v_cache.shape[2:])[slots] = v[ok].to(v_cache.dtype)


def linear_planes(x, w):
    """``linear`` for consumers that also accept the un-added K-slice planes of a GEMM (a kernel-side notion: here
    simply the product)."""
    return linear(x, w)


def mla_paged_decode(q, k_cache, lora, block_tables, seq_lens, scale):
    """Decode step of multi-head latent attention in the absorbed form: ``q`` [B, heads, lora + rope] (one query
    token per sequence) against the paged latent cache ``k_cache`` [blocks, block, 1, lora + rope]; the values are
    the latent part of the cached rows.  Returns [B, heads, lora]."""
    from chatlearn_b200.models.nn.mla import latent_paged_attention
    return latent_paged_attention(q, k_cache, lora, block_tables, seq_lens, None, 1, scale)


def paged_attention(q, k_cache, v_cache, block_tables, seq_lens, q_lens=None, scale=None, groups=None):
    """Attention of new queries against a paged KV cache (keys of the new tokens
    already appended).  ``q [Tq, nq, d]`` holds ``q_lens[b]`` trailing query
    tokens of each sequence ``b`` (1 each for decode); causal inside the tail.
    ``groups`` (which sequences share their first blocks) is a hint for the kernels:
    it changes how the work is split, not the result, and is ignored here."""
    B = seq_lens.shape[0]
    nb, bs, nkv, dk = k_cache.shape
    nq = q.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if q_lens is None:
        q_lens = torch.ones_like(seq_lens)
    outs, off = [], 0
    sl, ql = seq_lens.tolist(), q_lens.tolist()
    for b in range(B):
        L, nqt = sl[b], ql[b]
        if nqt == 0:
            continue
        nblk = (L + bs - 1) // bs
        blocks = block_tables[b, :nblk].long()
        kk = k_cache[blocks].reshape(nblk * bs, nkv, dk)[:L]
        vv = v_cache[blocks].reshape(nblk * bs, nkv, -1)[:L]
        qq = q[off:off + nqt]
        rep = nq // nkv
        kk = kk.repeat_interleave(rep, dim=1) if rep > 1 else kk
        vv = vv.repeat_interleave(rep, dim=1) if rep > 1 else vv
        att = torch.einsum("qhd,khd->hqk", qq.float(), kk.float()) * scale
        qpos = torch.arange(L - nqt, L, device=q.device)[:, None]
        kpos = torch.arange(L, device=q.device)[None, :]
        att = att.masked_fill((kpos > qpos)[None], float("-inf"))
        p = att.softmax(-1)
        outs.append(torch.einsum("hqk,khd->qhd", p, vv.float()).to(q.dtype))
        off += nqt
    return torch.cat(outs, 0)


# ------------------------------------------------------------------ lm head
class _LMHeadLogprob(torch.autograd.Function):
    """log p(label), entropy without keeping ``[T, V]`` logits: rows are processed
    in chunks and the backward recomputes each chunk's logits."""

    @staticmethod
    def forward(ctx, h, w, labels, inv_temp, chunk):
        T = h.shape[0]
        lp = torch.empty(T, dtype=torch.float32, device=h.device)
        ent = torch.empty(T, dtype=torch.float32, device=h.device)
        for s in range(0, T, chunk):
            z = (h[s:s + chunk] @ w.t()).float() * inv_temp
            lse = torch.logsumexp(z, -1)
            p = torch.exp(z - lse[:, None])
            lp[s:s + chunk] = z.gather(1, labels[s:s + chunk, None].long()).squeeze(1) - lse
            ent[s:s + chunk] = lse - (p * z).sum(-1)
        ctx.save_for_backward(h, w, labels)
        ctx.inv_temp, ctx.chunk = inv_temp, chunk
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        h, w, labels = ctx.saved_tensors
        inv_temp, chunk = ctx.inv_temp, ctx.chunk
        T = h.shape[0]
        gh = torch.empty_like(h)
        gw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        for s in range(0, T, chunk):
            hc = h[s:s + chunk]
            z = (hc @ w.t()).float() * inv_temp
            lse = torch.logsumexp(z, -1)
            p = torch.exp(z - lse[:, None])
            dz = -p * g_lp[s:s + chunk, None]
            dz.scatter_add_(1, labels[s:s + chunk, None].long(), g_lp[s:s + chunk, None].float())
            if g_ent is not None:
                pz = (p * z).sum(-1, keepdim=True)
                dz = dz - g_ent[s:s + chunk, None] * p * (z - pz)
            dz = (dz * inv_temp).to(h.dtype)
            gh[s:s + chunk] = dz @ w
            gw += (dz.t() @ hc).float()
        return gh, gw.to(w.dtype), None, None, None


def lmhead_logprob_entropy(h, w, labels, temperature: float = 1.0, chunk: int = 2048):
    """``h [T,H]``, ``w [V,H]``, ``labels [T]`` → (logprob ``[T]`` fp32, entropy ``[T]`` fp32)."""
    return _LMHeadLogprob.apply(h, w, labels, 1.0 / temperature, chunk)


def logprobs_from_logits(logits, labels):
    return torch.log_softmax(logits.float(), -1).gather(-1, labels.unsqueeze(-1).long()).squeeze(-1)


def entropy_from_logits(logits):
    z = logits.float()
    lse = torch.logsumexp(z, -1)
    return lse - (torch.softmax(z, -1) * z).sum(-1)


# ------------------------------------------------------------------ RL losses
def grpo_token_loss(logprobs, old_logprobs, advantages, pos_clip=0.2, neg_clip=0.2,
                    diff_clip=10.0, final_clip=3.0):
    """Clipped-ratio policy loss per token (chatlearn/algorithm/grpo_utils/loss_gallery.py:6-33)."""
    d = torch.clamp(logprobs - old_logprobs, max=diff_clip)
    ratio = torch.exp(d)
    adv = advantages if advantages.dim() == logprobs.dim() else advantages.unsqueeze(-1)
    l1 = -adv * ratio
    l2 = -adv * torch.clamp(ratio, 1.0 - neg_clip, 1.0 + pos_clip)
    return torch.clamp(torch.max(l1, l2), max=final_clip)


def gspo_token_loss(logprobs, old_logprobs, advantages, seq_ids, num_seqs, mask,
                    pos_clip=1e-3, neg_clip=1e-3, diff_clip=10.0, final_clip=3.0):
    """Group-sequence policy loss on a packed row (loss_gallery.py:35-74): the
    importance ratio is the masked sequence mean of the log-ratio, applied to each
    token through ``lp - sg(lp) + sg(mean)``."""
    m = mask.float()
    diff = (logprobs - old_logprobs) * m
    sums = torch.zeros(num_seqs, device=logprobs.device, dtype=torch.float32).index_add_(0, seq_ids, diff.float())
    cnt = torch.zeros(num_seqs, device=logprobs.device, dtype=torch.float32).index_add_(0, seq_ids, m)
    seq_mean = (sums / cnt.clamp(min=1.0)).detach()
    d = torch.clamp(logprobs - logprobs.detach() + seq_mean[seq_ids], max=diff_clip)
    ratio = torch.exp(d)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1.0 - neg_clip, 1.0 + pos_clip)
    loss = torch.clamp(torch.max(l1, l2), max=final_clip)
    with torch.no_grad():
        is_pos = (ratio > 1.0 + pos_clip) & (advantages > 0)
        is_neg = (ratio < 1.0 - neg_clip) & (advantages < 0)
    return loss, is_pos, is_neg


def gspo_loss_fused(logprobs, old_logprobs, ref_logprobs, advantages, mask, seq_ids, num_seqs, entropy=None,
                    pos_clip=3e-4, neg_clip=4e-4, diff_clip=10.0, final_clip=3.0,
                    kl_coef=0.0, entropy_coef=0.0, inv_norm=1.0):
    """Whole group-sequence (GSPO) loss of a packed row in one call: same contract as ``grpo_loss_fused``
    (``(total, stats)`` with ``stats = [pg_sum, kl_sum, ent_sum, clip_pos, clip_neg, n_tok]``)."""
    m = mask.float()
    adv = advantages if advantages.shape == logprobs.shape else advantages.expand_as(logprobs)
    pg, is_pos, is_neg = gspo_token_loss(logprobs, old_logprobs, adv, seq_ids, num_seqs, mask, pos_clip, neg_clip,
                                         diff_clip, final_clip)
    total = (pg * m).sum()
    stats = [(pg.detach() * m).sum()]
    if ref_logprobs is not None:
        kl = kl_k3(logprobs, ref_logprobs)
        total = total + kl_coef * (kl * m).sum()
        stats.append((kl.detach() * m).sum())
    else:
        stats.append(torch.zeros((), device=logprobs.device))
    if entropy is not None:
        total = total - entropy_coef * (entropy * m).sum()
        stats.append((entropy.detach() * m).sum())
    else:
        stats.append(torch.zeros((), device=logprobs.device))
    stats += [(is_pos.float() * m).sum(), (is_neg.float() * m).sum(), m.sum()]
    return total * inv_norm, torch.stack([t.float() for t in stats])


def kl_k3(logprobs, ref_logprobs):
    k = ref_logprobs - logprobs
    return torch.clamp(torch.exp(k) - k - 1.0, min=-10.0, max=10.0)


def grpo_loss_fused(logprobs, old_logprobs, ref_logprobs, advantages, mask, entropy=None,
                    pos_clip=0.2, neg_clip=0.2, diff_clip=10.0, final_clip=3.0,
                    kl_coef=0.0, entropy_coef=0.0, inv_norm=1.0):
    """Whole loss of a packed row in one call.

    Returns ``(total, stats)`` where total = Σ mask·(pg − c_ent·H + c_kl·KL)·inv_norm
    and ``stats`` = fp32 vector ``[pg_sum, kl_sum, ent_sum, clip_pos, clip_neg, n_tok]``."""
    m = mask.float()
    pg = grpo_token_loss(logprobs, old_logprobs, advantages, pos_clip, neg_clip, diff_clip, final_clip)
    total = (pg * m).sum()
    stats = [(pg.detach() * m).sum()]
    if ref_logprobs is not None:
        kl = kl_k3(logprobs, ref_logprobs)
        total = total + kl_coef * (kl * m).sum()
        stats.append((kl.detach() * m).sum())
    else:
        stats.append(torch.zeros((), device=logprobs.device))
    if entropy is not None:
        total = total - entropy_coef * (entropy * m).sum()
        stats.append((entropy.detach() * m).sum())
    else:
        stats.append(torch.zeros((), device=logprobs.device))
    with torch.no_grad():
        ratio = torch.exp(torch.clamp(logprobs - old_logprobs, max=diff_clip))
        stats.append(((ratio > 1 + pos_clip) & (advantages > 0)).float().mul(m).sum())
        stats.append(((ratio < 1 - neg_clip) & (advantages < 0)).float().mul(m).sum())
        stats.append(m.sum())
    return total * inv_norm, torch.stack([s.float() for s in stats])


# ------------------------------------------------------------------ optimizer
@torch.no_grad()
def adamw_step(master, grad, exp_avg, exp_avg_sq, out_param, step, lr, beta1, beta2, eps,
               weight_decay, grad_scale=1.0):
    """AdamW on an fp32 master shard; writes the updated weights to ``out_param``
    (compute dtype) as well.  ``grad_scale`` folds clip / unscale factors in."""
    g = grad.float() * grad_scale
    exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (exp_avg_sq / bc2).sqrt_().add_(eps)
    master.mul_(1 - lr * weight_decay).addcdiv_(exp_avg / bc1, denom, value=-lr)
    if out_param is not None:
        out_param.copy_(master)


@torch.no_grad()
def sumsq(x):
    return x.float().pow(2).sum()


# ------------------------------------------------------------------ MoE
def moe_router(logits, top_k, scoring="softmax", norm_topk=True, bias=None, n_group=1,
               topk_group=1, scale=1.0):
    """Router: scores → (group-limited) top-k → renormalised weights.

    Returns ``(weights [T,k] fp32, expert ids [T,k] int64, scores [T,E] fp32)``.
    ``bias`` only influences the selection (aux-loss-free balancing)."""
    z = logits.float()
    scores = torch.softmax(z, -1) if scoring == "softmax" else torch.sigmoid(z)
    sel = scores + bias.float() if bias is not None else scores
    T, E = sel.shape
    if n_group > 1:
        g = sel.view(T, n_group, E // n_group)
        gscore = g.topk(min(2, E // n_group), -1).values.sum(-1) if bias is not None else g.max(-1).values
        gidx = gscore.topk(topk_group, -1).indices
        gmask = torch.zeros(T, n_group, device=sel.device, dtype=torch.bool).scatter_(1, gidx, True)
        sel = sel.masked_fill(~gmask[:, :, None].expand(T, n_group, E // n_group).reshape(T, E),
                              float("-inf"))
    idx = sel.topk(top_k, -1).indices
    w = scores.gather(1, idx)
    if norm_topk:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * scale, idx, scores


def moe_aux_loss(scores, idx, num_experts, top_k):
    """Switch-style load-balancing loss: E · Σ_e f_e · P_e."""
    T = scores.shape[0]
    f = torch.zeros(num_experts, device=scores.device, dtype=torch.float32)
    f.index_add_(0, idx.reshape(-1), torch.ones(idx.numel(), device=scores.device))
    f = f / (T * top_k)
    P = scores.mean(0)
    return num_experts * (f * P).sum()


def grouped_mlp(xs, w13, w2, counts):
    """Expert MLPs over rows already sorted by expert: rows
    ``[sum(counts[:e]), sum(counts[:e+1]))`` go through expert ``e``.
    ``w13 [E, 2F, H]`` (gate rows then up rows), ``w2 [E, H, F]``; ``counts`` is a
    host list of length E."""
    outs, s = [], 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        h = swiglu(xs[s:s + n] @ w13[e].t())
        outs.append(h @ w2[e].t())
        s += n
    if not outs:
        return xs.new_zeros(0, w2.shape[1])
    return torch.cat(outs, 0)


def moe_experts(x, w13, w2, weights, idx):
    """Routed expert MLPs for tokens ``x [T,H]`` with ``weights/idx [T,k]``:
    sort (token, slot) pairs by expert, grouped MLP, fp32 weighted combine."""
    T, H = x.shape
    E = w13.shape[0]
    k = idx.shape[1]
    flat_e = idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = order // k
    counts = torch.bincount(flat_e, minlength=E).tolist()
    ys = grouped_mlp(x.index_select(0, tok), w13, w2, counts)
    wflat = weights.reshape(-1).index_select(0, order)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    out = out.index_add(0, tok, ys.float() * wflat[:, None].float())
    return out.to(x.dtype)


# ------------------------------------------------------------------ sampling
@torch.no_grad()
def sample(logits, u, temperature=1.0, top_k=-1, top_p=1.0, min_p=0.0):
    """Inverse-CDF sampling from filtered softmax.  ``logits [B,V]``, ``u [B]`` in
    [0,1).  Filters keep every token whose probability is ≥ the k-th largest /
    inside the smallest set reaching ``top_p`` mass / ≥ ``min_p·max``; ties at a
    threshold are kept.  ``temperature == 0`` is greedy.  Returns ``(ids, logprob
    under the unfiltered temperature-scaled distribution)``."""
    z = logits.float()
    if temperature == 0.0:
        ids = z.argmax(-1)
        return ids, torch.log_softmax(z, -1).gather(1, ids[:, None]).squeeze(1)
    z = z / temperature
    logp = torch.log_softmax(z, -1)
    p = logp.exp()
    keep = torch.ones_like(p, dtype=torch.bool)
    if top_k is not None and 0 < top_k < p.shape[-1]:
        kth = p.topk(top_k, -1).values[:, -1:]
        keep &= p >= kth
    if top_p < 1.0:
        sp, si = p.sort(-1, descending=True)
        cs = sp.cumsum(-1)
        # smallest prefix with mass >= top_p: keep entries whose preceding mass < top_p
        cut = (cs - sp) < top_p
        thr = torch.where(cut, sp, torch.full_like(sp, 2.0)).min(-1, keepdim=True).values
        keep &= p >= thr
    if min_p > 0.0:
        keep &= p >= min_p * p.max(-1, keepdim=True).values
    pf = torch.where(keep, p, torch.zeros_like(p))
    cdf = pf.cumsum(-1)
    target = u.float()[:, None] * cdf[:, -1:]
    ids = (cdf <= target).sum(-1).clamp(max=p.shape[-1] - 1)
    # never return a filtered-out token because of rounding at the boundary
    bad = ~keep.gather(1, ids[:, None]).squeeze(1)
    if bad.any():
        ids = torch.where(bad, pf.argmax(-1), ids)
    return ids, logp.gather(1, ids[:, None]).squeeze(1)


@torch.no_grad()
def apply_penalties(logits, token_counts, presence=0.0, frequency=0.0, repetition=1.0,
                    prompt_mask=None):
    """OpenAI-style presence/frequency penalties over generated-token counts and
    the multiplicative repetition penalty over prompt ∪ generated tokens."""
    z = logits.float()
    if repetition != 1.0:
        seen = token_counts > 0
        if prompt_mask is not None:
            seen = seen | prompt_mask
        z = torch.where(seen, torch.where(z > 0, z / repetition, z * repetition), z)
    if frequency != 0.0:
        z = z - frequency * token_counts.float()
    if presence != 0.0:
        z = z - presence * (token_counts > 0).float()
    return z
