"""Tensor-parallel pieces that are not plain linear layers.

``vocab_parallel_logprob_entropy``: per-token log p(label) and entropy when the LM
head is sharded over the vocabulary.  The reference computes the cross entropy
with Megatron's vocab-parallel loss and the entropy with three all-reduces of
``[T]`` (MAX, SUM, SUM; chatlearn/algorithm/grpo_utils/megatron_utils/train_helper.py:605-635).
Here every rank reduces its vocabulary shard to four numbers per token (local max,
sum-exp, sum-exp·z, label logit) and ONE all-gather of ``[T, 4]`` combines them;
``[T, V]`` logits exist only one row-chunk at a time.
"""
import torch

from chatlearn_b200 import ops
from .groups import Group


class _VocabParallelLogprob(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels, group: Group, vocab_start: int, inv_temp: float, chunk: int):
        T = h.shape[0]
        Vl = w.shape[0]
        loc = torch.empty(T, 4, dtype=torch.float32, device=h.device)
        local_label = labels - vocab_start
        mine = (local_label >= 0) & (local_label < Vl)
        safe = local_label.clamp(0, Vl - 1)
        for s in range(0, T, chunk):
            z = (h[s:s + chunk] @ w.t()).float() * inv_temp
            m = z.max(-1).values
            e = torch.exp(z - m[:, None])
            loc[s:s + chunk, 0] = m
            loc[s:s + chunk, 1] = e.sum(-1)
            loc[s:s + chunk, 2] = (e * z).sum(-1)
            zl = z.gather(1, safe[s:s + chunk, None]).squeeze(1)
            loc[s:s + chunk, 3] = torch.where(mine[s:s + chunk], zl, torch.zeros_like(zl))
        allv = group.all_gather_cat(loc.unsqueeze(0), 0)          # [tp, T, 4]
        M = allv[..., 0].max(0).values
        scale = torch.exp(allv[..., 0] - M[None])
        S = (allv[..., 1] * scale).sum(0)
        Tz = (allv[..., 2] * scale).sum(0)
        zl = allv[..., 3].sum(0)
        lse = M + torch.log(S)
        lp = zl - lse
        ent = lse - Tz / S
        ctx.save_for_backward(h, w, safe, mine, lse, ent)
        ctx.inv_temp, ctx.chunk = inv_temp, chunk
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        h, w, safe, mine, lse, ent = ctx.saved_tensors
        inv_temp, chunk = ctx.inv_temp, ctx.chunk
        T = h.shape[0]
        gh = torch.empty_like(h)
        gw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        pz = lse - ent
        for s in range(0, T, chunk):
            hc = h[s:s + chunk]
            z = (hc @ w.t()).float() * inv_temp
            p = torch.exp(z - lse[s:s + chunk, None])
            dz = -p * g_lp[s:s + chunk, None]
            if g_ent is not None:
                dz = dz - g_ent[s:s + chunk, None] * p * (z - pz[s:s + chunk, None])
            add = torch.where(mine[s:s + chunk], g_lp[s:s + chunk], torch.zeros_like(g_lp[s:s + chunk]))
            dz.scatter_add_(1, safe[s:s + chunk, None], add[:, None].float())
            dz = (dz * inv_temp).to(h.dtype)
            gh[s:s + chunk] = dz @ w          # partial over the vocabulary shard: summed by copy_in upstream
            gw += (dz.t() @ hc).float()
        return gh, gw.to(w.dtype), None, None, None, None, None


def vocab_parallel_logprob_entropy(h, w_local, labels, group: Group, temperature: float = 1.0,
                                   chunk: int = 2048):
    """``h [T,H]`` (replicated over the TP group), ``w_local [V/tp, H]``."""
    if group is None or group.size == 1:
        return ops.lmhead_logprob_entropy(h, w_local, labels, temperature, chunk)
    if torch.is_grad_enabled() and h.requires_grad:
        h = group.copy_in(h)
    vocab_start = group.rank * w_local.shape[0]
    return _VocabParallelLogprob.apply(h, w_local, labels.long(), group, vocab_start, 1.0 / temperature, chunk)
