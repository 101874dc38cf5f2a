"""Decode attention over the paged cache on batched PyTorch statements, without host synchronisation.

Serves head sizes the paged-decode kernels have no instance for (e.g. 256 for Qwen3-Next's attention
layers) so that such models still decode inside a captured CUDA graph: the block table gathers every
sequence's rows (padded to the table's width and masked by length), grouped-query heads attend to
their key head without repeating it.
"""
import torch


def paged_decode_batched(q, k_cache, v_cache, block_tables, seq_lens, scale: float):
    """``q`` [B, heads, dk], one new token per sequence whose key/value is already in the cache;
    caches [blocks, block, kv heads, d]; ``seq_lens`` [B] lengths including the new token."""
    B, nq, dk = q.shape
    nkv = k_cache.shape[2]
    rep = nq // nkv
    bt = block_tables.long()
    K = k_cache[bt].reshape(B, -1, nkv, dk)                    # [B, rows, kv heads, dk]
    V = v_cache[bt].reshape(B, K.shape[1], nkv, -1)
    qg = q.view(B, nkv, rep, dk).to(K.dtype)
    att = torch.einsum("bgrd,bkgd->bgrk", qg, K).float() * scale
    dead = torch.arange(K.shape[1], device=q.device)[None] >= seq_lens[:, None].long()
    p = att.masked_fill(dead[:, None, None], float("-inf")).softmax(-1).to(V.dtype)
    return torch.einsum("bgrk,bkgd->bgrd", p, V).reshape(B, nq, -1).to(q.dtype)
