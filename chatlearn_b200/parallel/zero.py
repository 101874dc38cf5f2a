"""Sharded training state (ZeRO / FSDP2-style) over flat parameter blocks.

The reference wraps HF models with torch ``fully_shard`` per decoder layer: bf16
parameters all-gathered before every layer forward and backward, fp32 gradients
reduce-scattered after every layer backward, AdamW on fp32 shards
(chatlearn/models/fsdp_module.py:356-394).  This is a re-design for 180 GB GPUs:

* compute-dtype parameters of every block stay resident and whole on each rank
  (Qwen3-8B bf16 = 16 GB), so forward/backward need no per-layer all-gather;
* gradients of all micro-batches of an optimizer step accumulate locally into
  one flat buffer per block and are reduce-scattered **once per step**;
* fp32 master weights and Adam moments exist only for this rank's 1/dp shard;
  after the update the new compute-dtype shard is all-gathered back into the
  resident parameters (or, with ``reshard=True``, gathered on demand per block
  — the memory-lean mode for models that do not fit).

Per optimizer step this moves 1 reduce-scatter + 1 all-gather of the model
instead of (2 all-gathers + 1 reduce-scatter) × micro-batches.  The collectives
are issued per block so they can overlap the backward of earlier blocks and the
update of later ones; the fused NVLink kernels (reduce-scatter + AdamW on the
owned shard, all-gather of the cast result) plug in through ``Group.fast``.
"""
from typing import Dict, List, Optional

import torch

from chatlearn_b200 import ops
from chatlearn_b200.models.nn.model import CausalLM, ParamBlock
from .groups import Group, single_group


class BlockState:
    """Optimizer-side state of one parameter block on one rank."""

    def __init__(self, block: ParamBlock, group: Group, grad_dtype, device, trainable=True):
        self.block, self.group = block, group
        n = block.numel
        assert n % group.size == 0, f"block {block.name}: {n} elements not divisible by {group.size}"
        self.shard_numel = n // group.size
        r = max(group.rank, 0)
        self.lo, self.hi = r * self.shard_numel, (r + 1) * self.shard_numel
        self.master = self.exp_avg = self.exp_avg_sq = self.grad = self.grad_shard = None
        if trainable:
            self.master = block.flat[self.lo:self.hi].float().clone()
            self.exp_avg = torch.zeros_like(self.master)
            self.exp_avg_sq = torch.zeros_like(self.master)
            self.grad = torch.zeros(n, dtype=grad_dtype, device=device)
            # a group of one owns the whole block: the fp32 accumulation buffer *is* the shard
            self.grad_shard = self.grad if (group.size == 1 and grad_dtype == torch.float32) else \
                torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
            block.enable_grad(self.grad)


class ShardedTrainState:
    def __init__(self, model: CausalLM, dp_group: Optional[Group] = None,
                 expert_dp_group: Optional[Group] = None, lr=2e-6, betas=(0.9, 0.95), eps=1e-8,
                 weight_decay=0.01, clip_grad=1.0, grad_dtype=torch.float32,
                 extra_norm_groups: Optional[List[Group]] = None, tp_size: int = 1,
                 ep_group: Optional[Group] = None, tp_group: Optional[Group] = None,
                 replica_group: Optional[Group] = None):
        self.model = model
        # hybrid sharding (HSDP): ``dp_group`` is the shard group (one node, say); the ranks with the same shard
        # in the other shard groups form ``replica_group`` and sum their gradient shards after the reduce-scatter,
        # so parameters are gathered inside the shard group only
        self.replica = replica_group if (replica_group is not None and replica_group.size > 1) else None
        # weight of a block's squared gradient norm in the global norm: below 1 for a block of which several
        # pipeline stages hold copies (tied embeddings on the first and the last stage)
        self.block_norm_weight: Dict[str, float] = {}
        self.tp_size, self.ep_group, self.tp_group = tp_size, ep_group, tp_group
        # expert tensor parallelism: the expert leaves of the tensor-parallel ranks are different slices
        self.expert_tp_sharded = getattr(model, "etp", 1) > 1
        self.dp = dp_group or single_group()
        self.edp = expert_dp_group or self.dp
        self.lr, self.betas, self.eps, self.wd, self.clip = lr, betas, eps, weight_decay, clip_grad
        self.step_count = 0
        # groups over which the squared grad norm must still be summed after the DP
        # shards are combined (tensor / expert / pipeline model parallel groups)
        self.extra_norm_groups = extra_norm_groups or []
        self.states: List[BlockState] = []
        for b in model.blocks:
            g = self.edp if b.name.endswith(".experts") else self.dp
            self.states.append(BlockState(b, g, grad_dtype, model.device))
        self.last_grad_norm = 0.0
        self.symm = None            # parallel.symm_collectives.SymmGroup once enable_symm() succeeded

    # ------------------------------------------------------------------ in-kernel collectives
    def enable_symm(self) -> bool:
        """Move the parameters and gradient buffers of the data-parallel blocks into
        symmetric memory, so that the optimizer step runs as two peer-memory kernels per
        block (pull reduce-scatter + squared norm; AdamW + push all-gather) instead of
        NCCL reduce-scatter / all-gather.  Collective over the data-parallel group;
        returns False (and changes nothing) where symmetric memory is unavailable.
        Buffers in symmetric memory stay resident: they are never offloaded or freed."""
        from . import symm_collectives, symm_mem
        dp = self.dp
        dev = self.model.device
        if dev.type != "cuda" or dp.size < 2 or dp.size > 8 or self.tp_size != 1:
            return False
        mine = [s for s in self.states if s.group is dp and s.grad is not None]
        if not mine or any(s.grad.dtype != torch.float32 or s.shard_numel % 4 or s.lo % 4 for s in mine):
            return False
        sg = symm_collectives.get(dp)
        if sg is None:
            return False
        total = sum(s.block.numel for s in mine)
        pdt = mine[0].block.flat.dtype
        p_arena = symm_mem.empty(total, pdt, dev, group=dp.pg)
        g_arena = symm_mem.empty(total, torch.float32, dev, group=dp.pg)
        g_arena.zero_()
        off = 0
        for s in mine:
            n = s.block.numel
            flat = p_arena[off:off + n]
            flat.copy_(s.block.flat)
            s.block.bind(flat)
            s.grad = g_arena[off:off + n]
            s.block.enable_grad(s.grad)
            s.grad_shard = torch.zeros(s.shard_numel, dtype=torch.float32, device=dev)
            s.symm = True
            off += n
        self._arenas = (p_arena, g_arena)
        torch.cuda.synchronize(dev)
        dp.barrier()
        self.symm = sg
        return True

    # ------------------------------------------------------------------ step
    def zero_grad(self):
        for s in self.states:
            s.grad.zero_()

    @torch.no_grad()
    def reduce_grads(self):
        """Reduce-scatter every block's accumulated gradient into its fp32 shard."""
        for s in self.states:
            if self.tp_group is not None and self.tp_group.size > 1:
                # leaves shared by tensor-sharded heads hold partial sums: complete them first
                for lf in s.block.leaves:
                    if getattr(lf, "grad_sum_tp", False):
                        o = s.block.offsets[lf.name]
                        self.tp_group.all_reduce_(s.grad[o:o + lf.numel])
                    kv = getattr(lf, "grad_sum_kv", None)
                    if kv is not None:
                        # key/value heads held by several ranks: every rank puts its rows into the slot of its head,
                        # the sum over the group completes each head's gradient
                        r0, n, head, heads = kv
                        o = s.block.offsets[lf.name]
                        rows = s.grad[o:o + lf.numel].view(lf.matrix_shape)[r0:r0 + n]
                        buf = rows.new_zeros((heads,) + tuple(rows.shape))
                        buf[head].copy_(rows)
                        self.tp_group.all_reduce_(buf)
                        rows.copy_(buf[head])
            g = s.group
            fused = g.fast.get("reduce_scatter_f32")
            if self.symm is not None and getattr(s, "symm", False):
                # every rank pulls its shard from all peers' gradient buffers over NVLink and
                # sums it; the kernel also leaves the shard's squared norm (per-CTA partials)
                s.sq_partial = self.symm.reduce_scatter_pull(s.grad, s.grad_shard, s.lo)
            elif fused is not None and s.grad.is_cuda:
                fused(s.grad_shard, s.grad)
            elif g.size == 1:
                if s.grad_shard.data_ptr() != s.grad.data_ptr():
                    s.grad_shard.copy_(s.grad)
            else:
                src = s.grad if s.grad.dtype == torch.float32 else s.grad.float()
                g.reduce_scatter_flat(s.grad_shard, src)
            if self.replica is not None and g is self.dp:
                self.replica.all_reduce_(s.grad_shard)
                s.sq_partial = None          # the squared norm a fused reduce-scatter left predates this sum

    @torch.no_grad()
    def _norm_ranges(self, s: "BlockState"):
        """(start, end, weight) pieces of a block's shard for the squared norm: leaves
        replicated over the tensor-parallel group carry weight 1/tp so that the sum over
        that group counts them once."""
        cached = getattr(s, "_norm_ranges", None)
        if cached is not None:
            return cached
        share = self.block_norm_weight.get(s.block.name, 1.0)     # a block that several pipeline stages hold
        if self.tp_size == 1:
            out = [(0, s.shard_numel, share)]
        else:
            out = []
            for lf in s.block.leaves:
                o = s.block.offsets[lf.name]
                if s.block.name.endswith(".experts"):
                    # with an expert-data-parallel group of their own they are summed over the expert-parallel
                    # group instead (below); otherwise the tensor-parallel ranks hold copies of the same experts
                    # unless expert tensor parallelism slices them
                    own = s.group is self.edp and self.edp is not self.dp
                    rep = not own and not self.expert_tp_sharded
                else:
                    rep = lf.replicated
                w = (1.0 / self.tp_size if rep else 1.0) * share
                pieces = [(o, o + lf.numel, w)]
                kv = getattr(lf, "grad_sum_kv", None)
                if kv is not None:
                    # rows of key/value heads that tp / heads ranks hold: counted once per head
                    cols = lf.matrix_shape[1]
                    k0, k1 = o + kv[0] * cols, o + (kv[0] + kv[1]) * cols
                    pieces = [(o, k0, w), (k0, k1, share * kv[3] / self.tp_size), (k1, o + lf.numel, w)]
                for p0, p1, pw in pieces:
                    a, b = max(p0, s.lo), min(p1, s.hi)
                    if b <= a:
                        continue
                    if out and out[-1][2] == pw and out[-1][1] == a - s.lo:
                        out[-1] = (out[-1][0], b - s.lo, pw)
                    else:
                        out.append((a - s.lo, b - s.lo, pw))
        s._norm_ranges = out
        return out

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the reduced gradient: shards are summed over their
        data-parallel group, expert shards additionally over the expert-parallel group,
        then everything over the tensor / pipeline groups (replicated leaves once)."""
        dev = self.model.device
        dp_sq = torch.zeros((), dtype=torch.float32, device=dev)
        edp_sq = torch.zeros((), dtype=torch.float32, device=dev)
        for s in self.states:
            v = torch.zeros((), dtype=torch.float32, device=dev)
            if getattr(s, "sq_partial", None) is not None:
                v = s.sq_partial.sum()        # computed by the reduce-scatter kernel
                s.sq_partial = None
            else:
                for a, b, w in self._norm_ranges(s):
                    v = v + ops.sumsq(s.grad_shard[a:b]) * w
            if s.group is self.edp and self.edp is not self.dp:
                edp_sq += v
            else:
                dp_sq += v
        # dense leaves: shards over dp, then the tensor- and pipeline-parallel groups;
        # expert leaves: shards over expert-dp, then the expert- and pipeline-parallel
        # groups (never the tensor group: expert weights are not tensor-sharded)
        self.dp.all_reduce_(dp_sq)
        for g in self.extra_norm_groups:
            g.all_reduce_(dp_sq)
        if self.edp is not self.dp:
            self.edp.all_reduce_(edp_sq)
            if self.ep_group is not None:
                self.ep_group.all_reduce_(edp_sq)
            for g in self.extra_norm_groups:
                if g is not self.tp_group or self.expert_tp_sharded:
                    g.all_reduce_(edp_sq)
        return (dp_sq + edp_sq).sqrt()

    @torch.no_grad()
    def step(self, lr: Optional[float] = None) -> float:
        """reduce → clip → AdamW on the shard → all-gather the new parameters."""
        self.reduce_grads()
        norm = self.grad_norm()
        self.last_grad_norm = norm
        scale = 1.0
        if self.clip and self.clip > 0:
            # stays on device: no host sync between the norm and the update
            scale = torch.clamp(self.clip / (norm + 1e-6), max=1.0)
        self.step_count += 1
        lr = self.lr if lr is None else lr
        for s in self.states:
            if self.symm is not None and getattr(s, "symm", False):
                # AdamW on the shard; the new weights are stored straight into every rank's
                # parameter buffer (the all-gather), completion is agreed inside the kernel
                self.symm.adamw_push(s.master, s.grad_shard, s.exp_avg, s.exp_avg_sq, s.block.flat, s.lo,
                                     self.step_count, lr, self.betas[0], self.betas[1], self.eps, self.wd,
                                     scale if torch.is_tensor(scale) else None)
                continue
            new_shard = s.block.flat[s.lo:s.hi]
            ops.adamw_step(s.master, s.grad_shard, s.exp_avg, s.exp_avg_sq, new_shard,
                           self.step_count, lr, self.betas[0], self.betas[1], self.eps, self.wd,
                           scale)
            if s.group.size > 1:
                fused = s.group.fast.get("all_gather")
                if fused is not None and new_shard.is_cuda:
                    fused(s.block.flat, new_shard)
                else:
                    s.group.all_gather_flat(s.block.flat, new_shard.clone())
        return norm

    @torch.no_grad()
    def rebuild_params(self):
        """Re-create the compute-dtype parameters from the fp32 master shards (cast, then all-gather):
        what the last optimizer step wrote, bit for bit."""
        for s in self.states:
            if s.master is None:
                continue
            new_shard = s.block.flat[s.lo:s.hi]
            new_shard.copy_(s.master)
            if s.group.size > 1:
                s.group.all_gather_flat(s.block.flat, new_shard.clone())

    # ------------------------------------------------------------------ residency
    def tensors_for(self, tag: str) -> List[List]:
        """(owner object, attribute) pairs of the tensors behind a memory tag."""
        out = []
        for s in self.states:
            if getattr(s, "symm", False) and tag in ("weights", "grads"):
                continue                      # symmetric-memory buffers stay resident
            if tag == "weights":
                out.append((s.block, "flat"))
            elif tag == "grads":
                out.extend([(s, "grad"), (s, "grad_shard")])
            elif tag == "optimizer":
                out.extend([(s, "master"), (s, "exp_avg"), (s, "exp_avg_sq")])
        return out

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self) -> Dict:
        return {
            "step": self.step_count,
            "blocks": {s.block.name: {"master": s.master.cpu(), "exp_avg": s.exp_avg.cpu(),
                                      "exp_avg_sq": s.exp_avg_sq.cpu(), "lo": s.lo, "hi": s.hi,
                                      "numel": s.block.numel} for s in self.states},
        }

    @torch.no_grad()
    def load_state_dict(self, sd: Dict):
        self.step_count = sd["step"]
        for s in self.states:
            b = sd["blocks"][s.block.name]
            assert (b["lo"], b["hi"]) == (s.lo, s.hi), "checkpoint was written with another dp size"
            s.master.copy_(b["master"])
            s.exp_avg.copy_(b["exp_avg"])
            s.exp_avg_sq.copy_(b["exp_avg_sq"])
            s.block.flat[s.lo:s.hi].copy_(s.master)
            if s.group.size > 1:
                s.group.all_gather_flat(s.block.flat, s.block.flat[s.lo:s.hi].clone())
