"""Expert parallelism: all-to-all token dispatch → local grouped expert MLP →
all-to-all combine.

The reference uses Megatron-Core's ``alltoall`` token dispatcher with
TransformerEngine ``moe_permute`` / grouped GEMM / ``moe_unpermute``
(chatlearn/models/patches/transformers/layers/groupgemm.py:40-211,
chatlearn/utils/megatron_utils.py:59-63).  This is the NCCL statement of that
path (also the CPU/gloo path); the fused in-kernel variant writes tokens
straight into the owning rank's expert buffers over NVLink and registers itself
as ``group.fast["moe_dispatch_combine"]``.
"""
import torch

from chatlearn_b200 import ops
from .groups import Group


class ExpertParallel:
    def __init__(self, group: Group):
        self.group = group
        self.size, self.rank = group.size, group.rank

    def experts(self, x, w13, w2, weights, idx, num_experts: int):
        """``x [T,H]``; ``w13/w2`` hold this rank's ``E/ep`` experts; ``idx`` are
        global expert ids.  Returns the combined expert output ``[T,H]``."""
        fast = self.group.fast.get("moe_dispatch_combine")
        if fast is not None and x.is_cuda and not torch.is_grad_enabled() and x.dtype == torch.bfloat16:
            return fast(x, w13, w2, weights, idx, num_experts)
        ep = self.size
        El = num_experts // ep
        T, H = x.shape
        k = idx.shape[1]
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)          # sorted by (dest rank, local expert)
        tok = order // k
        counts = torch.bincount(flat_e, minlength=num_experts)       # [E]
        # exchange per-expert counts: recv_counts[r, j] = rows rank r sends for my expert j
        recv_counts = self.group.all_to_all_single(counts.view(ep, El).contiguous())
        send_splits = counts.view(ep, El).sum(1).tolist()
        recv_mat = recv_counts.view(ep, El)
        recv_splits = recv_mat.sum(1).tolist()
        xs = self.group.all_to_all(x.index_select(0, tok), recv_splits, send_splits)
        # received rows are ordered (source rank, local expert): regroup by expert
        rm = recv_mat.tolist()
        exp_of_row = torch.cat([torch.full((rm[r][j],), j, dtype=torch.long)
                                for r in range(ep) for j in range(El)]).to(x.device) \
            if sum(recv_splits) else torch.zeros(0, dtype=torch.long, device=x.device)
        regroup = torch.argsort(exp_of_row, stable=True)
        per_expert = recv_mat.sum(0).tolist()
        ys = ops.grouped_mlp(xs.index_select(0, regroup), w13, w2, per_expert)
        inv = torch.empty_like(regroup)
        inv[regroup] = torch.arange(regroup.numel(), device=x.device)
        ys = ys.index_select(0, inv)
        back = self.group.all_to_all(ys, send_splits, recv_splits)
        wflat = weights.reshape(-1).index_select(0, order)
        out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
        out = out.index_add(0, tok, back.float() * wflat[:, None].float())
        return out.to(x.dtype)
