"""Context parallelism: zig-zag sequence split, KV all-gather into local memory,
then local attention.

The reference delegates CP attention to Megatron-Core/TransformerEngine and owns
only the batch split and the log-prob re-gather
(chatlearn/algorithm/grpo_utils/megatron_utils/train_helper.py:194-230,257-327).
Here every sequence of the packed row is padded to a multiple of ``2·cp`` and cut
into ``2·cp`` chunks; rank ``r`` keeps chunks ``r`` and ``2·cp-1-r`` (balanced causal
work).  K and V are all-gathered (the cheap tensors under GQA/MLA), reordered to
sequence order, and each local query chunk attends to its causal prefix.
"""
from typing import List

import torch

from chatlearn_b200 import ops
from .groups import Group


def zigzag_indices(seq_lens: List[int], cp: int, rank: int) -> torch.Tensor:
    """Indices into the (padded) packed row owned by ``rank``."""
    out, off = [], 0
    for L in seq_lens:
        assert L % (2 * cp) == 0, "sequences must be padded to a multiple of 2*cp"
        c = L // (2 * cp)
        out.append(torch.arange(off + rank * c, off + (rank + 1) * c))
        out.append(torch.arange(off + (2 * cp - 1 - rank) * c, off + (2 * cp - rank) * c))
        off += L
    return torch.cat(out) if out else torch.zeros(0, dtype=torch.long)


def pad_to_multiple(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class ContextParallel:
    def __init__(self, group: Group):
        self.group = group
        self.size, self.rank = group.size, group.rank
        self._plan_key, self._plan = None, None

    def plan(self, seq_lens: List[int], device):
        """Host-side index plan for a packed row (cached per seq_lens)."""
        key = tuple(seq_lens)
        if key == self._plan_key:
            return self._plan
        cp = self.size
        # position of every global token in the rank-major gathered buffer
        per_rank = [zigzag_indices(seq_lens, cp, r) for r in range(cp)]
        Tl = per_rank[0].numel()
        total = sum(seq_lens)
        inv = torch.empty(total, dtype=torch.long)
        for r, idx in enumerate(per_rank):
            inv[idx] = torch.arange(Tl) + r * Tl
        q_starts, q_lens, k_starts, k_lens = [], [], [], []
        off_local, off_glob = 0, 0
        for L in seq_lens:
            c = L // (2 * cp)
            for chunk in (self.rank, 2 * cp - 1 - self.rank):
                q_starts.append(off_local)
                q_lens.append(c)
                k_starts.append(off_glob)
                k_lens.append((chunk + 1) * c)
                off_local += c
            off_glob += L
        mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)  # noqa: E731
        self._plan_key = key
        self._plan = dict(inv=inv.to(device), local=per_rank[self.rank].to(device),
                          q_starts=mk(q_starts), q_lens=mk(q_lens), k_starts=mk(k_starts),
                          k_lens=mk(k_lens), max_q=max(q_lens) if q_lens else 0,
                          max_k=max(k_lens) if k_lens else 0, seq_lens=list(seq_lens))
        return self._plan

    def attention(self, q, k, v, ctx, scale):
        plan = ctx.cp_plan
        kf = self.group.gather_sum_bwd(k).index_select(0, plan["inv"])
        vf = self.group.gather_sum_bwd(v).index_select(0, plan["inv"])
        return ops.attention_segments(q, kf, vf, plan["q_starts"], plan["q_lens"],
                                      plan["k_starts"], plan["k_lens"], scale,
                                      plan["max_q"], plan["max_k"])

    def gather_tokens(self, x_local, plan):
        """Per-token values of all ranks in global sequence order (log-prob re-gather)."""
        return self.group.all_gather_cat(x_local.contiguous(), 0).index_select(0, plan["inv"])
