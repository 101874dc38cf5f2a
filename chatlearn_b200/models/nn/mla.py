"""Latent-space attention against the compressed cache of multi-head latent attention (MLA).

Every cached row is ``[normalised latent (kv_lora_rank) | rotary key (qk_rope_head_dim)]``, shared
by all heads.  With the key up-projection folded into the query and the value up-projection applied
after the attention, decode is a one-"head" attention whose keys are the cached rows and whose values
are their latent part (DeepSeek-V2/V3 "absorbed" form; the reference leaves this to vLLM/SGLang's MLA
backends, chatlearn/models/vllm_module.py:442-469 only sizes the cache).

Batched PyTorch statements without host synchronisation (safe inside a captured decode step): the
block table gathers each sequence's rows, masked by length; the keys are never repeated per head.
"""
import torch


def latent_paged_attention(q, k_cache, lora: int, block_tables, seq_lens, q_lens, max_q: int, scale: float):
    """``q`` [T, heads, lora + rope] (queries of all sequences, ``q_lens[b]`` trailing tokens of sequence b, one
    each when ``q_lens`` is None); ``k_cache`` [blocks, block, 1, lora + rope]; ``seq_lens`` [B] lengths including
    the new tokens.  Returns [T, heads, lora]."""
    T, nh, D = q.shape
    B = seq_lens.shape[0]
    bs = k_cache.shape[1]
    dev = q.device
    rows = k_cache[block_tables.long()].reshape(B, -1, D)                  # [B, K, D]; rows past the length are masked
    K = rows.shape[1]
    kpos = torch.arange(K, device=dev)
    if q_lens is None or max_q <= 1:
        assert T == B
        att = torch.bmm(q, rows.transpose(1, 2)).float() * scale            # [B, heads, K]
        att = att.masked_fill((kpos[None] >= seq_lens[:, None].long())[:, None], float("-inf"))
        p = att.softmax(-1).to(q.dtype)
        return torch.bmm(p, rows[..., :lora])
    ql = q_lens.long()
    seq = torch.repeat_interleave(torch.arange(B, device=dev), ql, output_size=T)
    off = torch.arange(T, device=dev) - (torch.cumsum(ql, 0) - ql)[seq]
    qp = q.new_zeros(B, max_q, nh, D)
    qp[seq, off] = q
    att = torch.bmm(qp.reshape(B, max_q * nh, D), rows.transpose(1, 2)).float().view(B, max_q, nh, K) * scale
    # query i of a tail of n tokens sits at position len - n + i and sees keys up to itself
    qpos = (seq_lens.long() - ql)[:, None] + torch.arange(max_q, device=dev)[None]
    att = att.masked_fill((kpos[None, None] > qpos[:, :, None])[:, :, None], float("-inf"))
    p = att.softmax(-1).to(q.dtype).view(B, max_q * nh, K)
    o = torch.bmm(p, rows[..., :lora]).view(B, max_q, nh, lora)
    return o[seq, off]


# ------------------------------------------------------------------ rotary embedding of the decoupled key
def yarn_mscale(factor: float, m: float = 1.0) -> float:
    import math
    return 0.1 * m * math.log(factor) + 1.0 if factor > 1 else 1.0


def yarn_inv_freq(dim: int, theta: float, sc: dict):
    """Inverse frequencies of the YaRN long-context rescaling and the factor applied to cos/sin: low
    frequencies are interpolated by ``factor``, high ones kept, with a linear ramp between the two
    correction dims (DeepSeek-V3's released configuration; the reference passes ``rotary_scaling_factor``
    / ``mscale`` to Megatron in chatlearn/utils/megatron_utils.py:100-140)."""
    import math
    factor = float(sc["factor"])
    orig = float(sc.get("original_max_position_embeddings", 4096))
    beta_fast, beta_slow = float(sc.get("beta_fast", 32)), float(sc.get("beta_slow", 1))
    mscale, mscale_all = sc.get("mscale"), sc.get("mscale_all_dim")
    att = yarn_mscale(factor, mscale) / yarn_mscale(factor, mscale_all) if mscale and mscale_all else yarn_mscale(factor)

    def corr(rot):
        return dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(theta))
    low, high = corr(beta_fast), corr(beta_slow)
    if sc.get("truncate", True):
        low, high = math.floor(low), math.ceil(high)
    low, high = max(low, 0), min(high, dim - 1)
    if low == high:
        high += 0.001
    pos = theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim)
    ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
    inv = (1.0 / (factor * pos)) * ramp + (1.0 / pos) * (1 - ramp)
    return inv, float(att)


def attention_scale(arch) -> float:
    """Softmax scale of an MLA layer; YaRN multiplies it by mscale(factor, mscale_all_dim)^2."""
    s = (arch.qk_nope_head_dim + arch.qk_rope_head_dim) ** -0.5
    sc = arch.rope_scaling
    if sc and sc.get("mscale_all_dim"):
        m = yarn_mscale(float(sc["factor"]), float(sc["mscale_all_dim"]))
        s *= m * m
    return s


def rope_decoupled(arch, x, positions):
    """Rotary embedding of the rotary slice of q or k: ``x`` [T, heads, rope dims].  Checkpoints of this
    family store the rotary dims as (even, odd) pairs; they are brought into the half-split order first."""
    from chatlearn_b200 import ops
    T, h, rp = x.shape
    if arch.rope_interleave:
        x = x.view(T, h, rp // 2, 2).transpose(-1, -2).reshape(T, h, rp)
    if not arch.rope_scaling:
        return ops.rope(x.contiguous(), positions, arch.rope_theta)
    inv, att = yarn_inv_freq(rp, arch.rope_theta, arch.rope_scaling)
    ang = positions.float()[:, None] * inv.to(x.device)[None]              # [T, rp / 2]
    cos, sin = (torch.cat([f, f], -1)[:, None] * att for f in (ang.cos(), ang.sin()))
    xf = x.float()
    rot = torch.cat([-xf[..., rp // 2:], xf[..., :rp // 2]], dim=-1)
    return (xf * cos + rot * sin).to(x.dtype)
