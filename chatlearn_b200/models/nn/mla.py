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
