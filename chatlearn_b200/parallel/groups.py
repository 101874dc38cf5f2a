"""Process-group wrappers with autograd-aware collectives.

The reference gets these from Megatron-Core ``mpu`` / torch FSDP2 / its own
Ulysses helpers (chatlearn/utils/communication_op.py:28-122).  Here a ``Group``
wraps one ``torch.distributed`` group (NCCL on GPUs, gloo on CPU ranks) and
exposes the collectives the model code needs, each as a differentiable function
with the correct conjugate collective in backward.  Fused in-kernel variants
(peer loads/stores over NVLink) register themselves on a group through
``Group.fast`` and take over for CUDA tensors.
"""
from typing import List, Optional

import torch
import torch.distributed as dist


def _backend(pg) -> str:
    return dist.get_backend(pg)


class Group:
    def __init__(self, pg, ranks: List[int], name: str = ""):
        self.pg, self.ranks, self.name = pg, list(ranks), name
        self.size = len(ranks)
        me = dist.get_rank() if dist.is_initialized() else 0
        self.rank = self.ranks.index(me) if me in self.ranks else -1
        self.fast = {}  # op name -> fused implementation (symmetric-memory kernels)

    @property
    def member(self):
        return self.rank >= 0

    # ---- raw (non-differentiable) collectives ----
    def all_reduce_(self, x, op=dist.ReduceOp.SUM):
        if self.size > 1:
            if "all_reduce" in self.fast and x.is_cuda and op == dist.ReduceOp.SUM:
                return self.fast["all_reduce"](x)
            dist.all_reduce(x, op=op, group=self.pg)
        return x

    def all_gather_cat(self, x, dim=0):
        """Concatenate equal-shaped ``x`` of all ranks along ``dim``."""
        if self.size == 1:
            return x
        x = x.contiguous()
        fast = self.fast.get("exchange") if x.is_cuda else None
        flat = fast.all_gather(x.view(-1)) if fast is not None else None
        if flat is not None:
            out = flat.view((self.size,) + tuple(x.shape))
            return out.reshape((-1,) + tuple(x.shape[1:])) if dim == 0 else torch.cat(list(out.unbind(0)), dim=dim)
        out = torch.empty((self.size,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out.view(-1), x.view(-1), group=self.pg) \
            if _backend(self.pg) == "nccl" else dist.all_gather(list(out.unbind(0)), x, group=self.pg)
        if dim == 0:
            return out.reshape((-1,) + tuple(x.shape[1:]))
        return torch.cat(list(out.unbind(0)), dim=dim)

    def all_gather_flat(self, out_flat, in_flat):
        if self.size == 1:
            out_flat.copy_(in_flat)
        elif _backend(self.pg) == "nccl":
            dist.all_gather_into_tensor(out_flat, in_flat, group=self.pg)
        else:
            dist.all_gather(list(out_flat.chunk(self.size)), in_flat, group=self.pg)
        return out_flat

    def reduce_scatter_flat(self, out_flat, in_flat, op=dist.ReduceOp.SUM):
        """``in_flat`` (size·n) → this rank's reduced chunk ``out_flat`` (n)."""
        if self.size == 1:
            out_flat.copy_(in_flat)
        elif _backend(self.pg) == "nccl":
            dist.reduce_scatter_tensor(out_flat, in_flat, op=op, group=self.pg)
        else:
            tmp = in_flat.clone()
            dist.all_reduce(tmp, op=op, group=self.pg)
            out_flat.copy_(tmp.chunk(self.size)[self.rank])
        return out_flat

    def all_to_all_single(self, x, out_splits=None, in_splits=None):
        """Rows of ``x`` are exchanged: rank r sends ``in_splits[j]`` rows to j."""
        if self.size == 1:
            return x
        x = x.contiguous()
        if out_splits is None and in_splits is None and x.is_cuda and "exchange" in self.fast:
            out = self.fast["exchange"].all_to_all(x)
            if out is not None:
                return out
        if out_splits is None:
            out = torch.empty_like(x)
        else:
            out = torch.empty((sum(out_splits),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        if _backend(self.pg) == "nccl":
            dist.all_to_all_single(out, x, out_splits, in_splits, group=self.pg)
        else:
            ins = list(x.split(in_splits if in_splits is not None else x.shape[0] // self.size))
            outs = list(out.split(out_splits if out_splits is not None else out.shape[0] // self.size))
            try:
                dist.all_to_all(outs, ins, group=self.pg)
            except RuntimeError:
                # gloo without all_to_all: pairwise exchange
                reqs = []
                for j in range(self.size):
                    if j == self.rank:
                        outs[j].copy_(ins[j])
                    else:
                        reqs.append(dist.isend(ins[j], self.ranks[j], group=self.pg))
                        reqs.append(dist.irecv(outs[j], self.ranks[j], group=self.pg))
                for r in reqs:
                    r.wait()
        return out

    def broadcast_(self, x, src_group_rank=0):
        if self.size > 1:
            dist.broadcast(x, self.ranks[src_group_rank], group=self.pg)
        return x

    def all_gather_object(self, obj):
        if self.size == 1:
            return [obj]
        out = [None] * self.size
        dist.all_gather_object(out, obj, group=self.pg)
        return out

    def barrier(self):
        if self.size > 1:
            dist.barrier(group=self.pg)

    # ---- differentiable collectives ----
    def all_reduce(self, x):
        """Sum over the group; gradient passes through unchanged (row-parallel output)."""
        return _AllReduce.apply(x, self) if self.size > 1 else x

    def copy_in(self, x):
        """Identity forward, all-reduce of the gradient (input of column-parallel layers)."""
        return _CopyIn.apply(x, self) if self.size > 1 else x

    def gather_seq(self, x, dim=0):
        """All-gather along ``dim``; backward keeps this rank's slice."""
        return _GatherSeq.apply(x, self, dim) if self.size > 1 else x

    def gather_sum_bwd(self, x):
        """All-gather along dim 0 (rank-major); backward reduce-scatters the gradient
        (used where every rank consumes the gathered tensor differently, e.g. CP K/V)."""
        return _GatherSumBwd.apply(x, self) if self.size > 1 else x

    def reduce_scatter_seq(self, x):
        """Sum over the group, keeping this rank's slice of dim 0; backward all-gathers the gradient
        (output of row-parallel layers under Megatron-style sequence parallelism)."""
        return _ReduceScatterSeq.apply(x, self) if self.size > 1 else x

    def scatter_seq(self, x):
        """This rank's slice of dim 0 of a tensor every rank holds whole; backward all-gathers the gradient
        (entry into a sequence-parallel region)."""
        return _ScatterSeq.apply(x, self) if self.size > 1 else x

    def all_to_all(self, x, out_splits=None, in_splits=None):
        return _AllToAll.apply(x, self, out_splits, in_splits) if self.size > 1 else x


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        return group.all_reduce_(x.clone() if x.requires_grad else x.contiguous())

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyIn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.group.all_reduce_(g.contiguous().clone()), None


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim, ctx.n = group, dim, x.shape[dim]
        return group.all_gather_cat(x, dim)

    @staticmethod
    def backward(ctx, g):
        r = ctx.group.rank
        return g.narrow(ctx.dim, r * ctx.n, ctx.n).contiguous(), None, None


class _GatherSumBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group, ctx.shape = group, x.shape
        return group.all_gather_cat(x, 0)

    @staticmethod
    def backward(ctx, g):
        out = torch.empty(ctx.shape, dtype=g.dtype, device=g.device)
        ctx.group.reduce_scatter_flat(out.view(-1), g.contiguous().view(-1))
        return out, None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        assert x.shape[0] % group.size == 0, f"{x.shape[0]} rows cannot be split over {group.size} ranks"
        out = torch.empty((x.shape[0] // group.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        group.reduce_scatter_flat(out.view(-1), x.contiguous().view(-1))
        return out

    @staticmethod
    def backward(ctx, g):
        return ctx.group.all_gather_cat(g.contiguous(), 0), None


class _ScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        assert x.shape[0] % group.size == 0, f"{x.shape[0]} rows cannot be split over {group.size} ranks"
        n = x.shape[0] // group.size
        return x.narrow(0, group.rank * n, n).contiguous()

    @staticmethod
    def backward(ctx, g):
        return ctx.group.all_gather_cat(g.contiguous(), 0), None


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, out_splits, in_splits):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        return group.all_to_all_single(x, out_splits, in_splits)

    @staticmethod
    def backward(ctx, g):
        return ctx.group.all_to_all_single(g, ctx.in_splits, ctx.out_splits), None, None, None


def single_group() -> Group:
    """Group of this process alone (no process group needed)."""
    g = Group.__new__(Group)
    g.pg, g.ranks, g.name, g.size, g.rank, g.fast = None, [0], "self", 1, 0, {}
    return g


def new_group(ranks: List[int], name: str = "", backend: Optional[str] = None) -> Group:
    """Collective over the whole world: every rank must call with the same args."""
    pg = dist.new_group(ranks=ranks, backend=backend)
    return Group(pg, ranks, name)
