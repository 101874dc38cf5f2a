"""In-kernel collectives over symmetric memory for one process group.

``SymmGroup`` owns the flag words and staging buffers of a group and exposes

* ``all_reduce(x)``      – one-shot all-reduce (every rank reads all peers' buffers and
  sums in a fixed order): the tensor-parallel all-reduce of the rollout decode step;
* ``reduce_scatter_pull`` / ``adamw_push`` – the two kernels of the sharded optimizer
  step: each rank *pulls* its gradient shard from every peer and sums it (plus the
  squared norm), then, once the clip factor is known, updates its fp32 shard and
  *pushes* the new bf16 weights into every peer's parameter buffer.

The reference uses NCCL collectives issued by torch FSDP2 / Megatron / vLLM for all
of these (chatlearn/models/fsdp_module.py:356-394); the NCCL path of
``parallel.groups`` stays as the baseline and the CPU/gloo implementation.
Synchronisation between ranks happens inside the kernels (flag words, bounded
waits); the host only launches.
"""
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from . import symm_mem
from .groups import Group

NUM_SLOTS = 1024          # barrier instances per sender (>= 2 x the largest grid)
PART_BYTES = 4 << 20      # each of the two buffers for un-reduced tensor-parallel partials


class SymmGroup:
    def __init__(self, group: Group, staging_bytes: int = 8 << 20):
        from chatlearn_b200.ops import native
        self.C = native.C
        self.native = native
        self.group = group
        self.rank, self.world = group.rank, group.size
        assert 1 < self.world <= 8
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.pg = group.pg
        # flag words: [sender rank][slot] uint32, zero-initialised, in symmetric memory
        self.flags = symm_mem.empty(8 * NUM_SLOTS, torch.int32, self.device, group=self.pg)
        self.flags.zero_()
        self.expect = torch.zeros(NUM_SLOTS * 8, dtype=torch.int32, device=self.device)
        self.flag_ptrs = self._ptrs(self.flags)
        self.staging = symm_mem.empty(staging_bytes // 2, torch.bfloat16, self.device, group=self.pg)
        self.staging_ptrs = self._ptrs(self.staging)
        # two buffers for row-parallel GEMM partials; consecutive calls alternate between them.
        # Each buffer has one slot per rank: rank r's GEMM epilogue stores its partial product into
        # slot r of EVERY rank's buffer (peer stores over NVLink), so the reduction reads local memory.
        self.slot_elems = PART_BYTES // 2
        self.parts = [symm_mem.empty(self.world * self.slot_elems, torch.bfloat16, self.device, group=self.pg)
                      for _ in range(2)]
        esz = 2
        self.push_ptrs = [[p + self.rank * self.slot_elems * esz for p in self._ptrs(t)] for t in self.parts]
        self.slot_ptrs = [[t.data_ptr() + r * self.slot_elems * esz for r in range(self.world)] for t in self.parts]
        # Measured on two B200 (decode step of 256 sequences, TP=2): pulling (K-sliced GEMM into the local
        # slot, reduction reads the peer) 13.1 ms; pushing from the GEMM epilogue (no K slicing possible,
        # stores cross NVLink) 13.8 ms.  Pull is the default; CLB200_TP_PUSH=1 selects the push epilogue.
        self.push = os.environ.get("CLB200_TP_PUSH", "0") == "1"
        self.part_ptrs = [self._ptrs(t) for t in self.parts]
        self._flip = 0
        self._xbufs, self._xptrs, self._xcap, self._xflip = None, None, 0, 0
        torch.cuda.synchronize()
        group.barrier()               # flags are zero everywhere before the first kernel signals

    def _ptrs(self, t: torch.Tensor) -> List[int]:
        return [symm_mem.peer_pointer(t, self.group.ranks[r]) for r in range(self.world)]

    # ------------------------------------------------------------------ all-reduce
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Sum ``x`` over the group.  ``x`` is copied into the staging buffer (unless it
        already lives there) and the result is written in place into ``x``."""
        n = x.numel()
        nbytes = n * x.element_size()
        if nbytes > self.staging.numel() * 2 or x.dtype not in (torch.bfloat16, torch.float32) or not x.is_contiguous():
            dist.all_reduce(x, group=self.pg)
            return x
        stage = self.staging.view(torch.uint8)[:nbytes].view(x.dtype)
        stage.copy_(x.view(-1))
        self.C.symm_allreduce(self.staging_ptrs, self.flag_ptrs, self.expect, x, n, self.rank, NUM_SLOTS)
        self.native.launch_counts["symm_allreduce"] += 1
        return x

    # ------------------------------------------------------------------ fused TP epilogue
    def fits(self, T: int, H: int) -> bool:
        return T * H * 2 <= PART_BYTES and H % 8 == 0 and H <= 8192

    def begin_forward(self):
        """Every forward pass issues an even number of partial/reduce pairs (two per layer),
        so the buffer alternation is the same in eager steps and in replayed CUDA graphs."""
        assert self._flip == 0, "odd number of tensor-parallel partial reductions in the last forward pass"

    def gemm_partial(self, x2d: torch.Tensor, w: torch.Tensor):
        """This rank's ``x2d @ w.T`` written into the next staging buffer; returns a handle
        for ``ar_residual_rmsnorm``."""
        idx = self._flip
        self._flip ^= 1
        T, N = x2d.shape[0], w.shape[0]
        base = self.rank * self.slot_elems
        out = self.parts[idx][base:base + T * N].view(T, N)           # my slot of my own buffer
        pushed = self.push and self.native.push_ok(x2d, w)        # same answer on every rank (same shapes)
        if T > 0:
            if pushed:
                self.native.linear_push(x2d, w, out, self.push_ptrs[idx])
            else:
                self.native.linear_out(x2d, w, out)
        return idx, out, pushed

    def ar_residual_rmsnorm(self, part, resid: torch.Tensor, w: Optional[torch.Tensor], eps: float):
        """``resid += sum over ranks of the partial``; returns ``rmsnorm(resid) * w`` (``None``
        when ``w`` is ``None``).  One kernel, peers read over NVLink."""
        idx, out, pushed = part
        assert out.shape == resid.shape
        self.native.launch_counts["symm_ar_residual_rmsnorm"] += 1
        # pushed partials: all slots are in local memory; otherwise read slot r from rank r's buffer
        ptrs = self.slot_ptrs[idx] if pushed else \
            [p + r * self.slot_elems * 2 for r, p in enumerate(self.part_ptrs[idx])]
        return self.C.symm_ar_residual_rmsnorm(ptrs, self.flag_ptrs, self.expect, resid, w,
                                               float(eps), self.rank, NUM_SLOTS)

    # ------------------------------------------------------------------ sharded optimizer step
    def symmetric_like(self, numel: int, dtype) -> torch.Tensor:
        return symm_mem.empty(numel, dtype, self.device, group=self.pg)

    def reduce_scatter_pull(self, grad_full: torch.Tensor, shard_out: torch.Tensor, lo: int) -> torch.Tensor:
        """``shard_out = sum over ranks of grad[lo:lo+len]``; returns partial sums of squares."""
        ptrs = self._ptrs(grad_full)
        part = self.C.symm_rs_pull_sumsq(ptrs, self.flag_ptrs, self.expect, shard_out, lo, self.rank, NUM_SLOTS)
        self.native.launch_counts["symm_rs_pull"] += 1
        return part

    def adamw_push(self, master, grad_shard, exp_avg, exp_avg_sq, param_full: torch.Tensor, lo: int, step: int,
                   lr, beta1, beta2, eps, wd, scale: Optional[torch.Tensor]):
        ptrs = self._ptrs(param_full)
        self.C.symm_adamw_push(master, grad_shard, exp_avg, exp_avg_sq, ptrs, self.flag_ptrs, self.expect, lo,
                               param_full.dtype == torch.bfloat16, int(step), lr, beta1, beta2, eps, wd,
                               scale.reshape(1).float() if scale is not None else None, self.rank, NUM_SLOTS)
        self.native.launch_counts["symm_adamw_push"] += 1

    # ------------------------------------------------------------------ all-gather / all-to-all
    def _exchange_buffers(self):
        """Two receive buffers per rank, used alternately: a peer writes into buffer ``i`` for call
        ``k+2`` only after the barrier of call ``k+1``, which this rank signals after it has copied
        the result of call ``k`` out, so one barrier per call is enough.  Allocated collectively on
        the first exchange of the group."""
        if self._xbufs is None:
            cap = int(os.environ.get("CLB200_SYMM_XCHG_MB", "192")) << 20
            self._xbufs = [symm_mem.empty(cap, torch.uint8, self.device, group=self.pg) for _ in range(2)]
            self._xptrs = [self._ptrs(t) for t in self._xbufs]
            self._xcap = cap
        return self._xbufs

    def _exchange(self, x: torch.Tensor, chunk_bytes: int, all_to_all: bool) -> Optional[torch.Tensor]:
        total = chunk_bytes * self.world
        if chunk_bytes == 0 or chunk_bytes % 16 or x.data_ptr() % 16 or not x.is_contiguous():
            return None
        bufs = self._exchange_buffers()
        if total > self._xcap:
            return None
        idx = self._xflip
        self._xflip ^= 1
        self.C.symm_push_chunks(x, self._xptrs[idx], chunk_bytes, all_to_all, self.rank)
        self.C.symm_group_barrier(self.flag_ptrs, self.expect, NUM_SLOTS - 1, NUM_SLOTS, self.rank)
        self.native.launch_counts["symm_exchange"] += 1
        return bufs[idx][:total].view(x.dtype).clone()

    def gemm_reduce_scatter(self, x2d: torch.Tensor, w: torch.Tensor) -> Optional[torch.Tensor]:
        """``reduce_scatter(x2d @ w.T)`` along the rows in one pass: the GEMM epilogue stores every row block of
        this rank's partial product straight into the receive buffer of the rank that owns the block (tile by
        tile, over NVLink, while the next tile is being multiplied), one flag barrier makes the chunks visible,
        and the owner adds its ``world`` chunks.  Output of a row-parallel layer under sequence parallelism
        (the reference leaves it to Megatron: GEMM, then an NCCL reduce-scatter).  ``None`` when the shapes do
        not qualify (the caller then multiplies and reduce-scatters separately)."""
        M, N = x2d.shape[0], w.shape[0]
        if M % self.world or M == 0 or not self.native.push_ok(x2d, w) or N % 8:
            return None
        rows = M // self.world
        chunk_bytes = rows * N * 2
        if chunk_bytes % 16:
            return None
        bufs = self._exchange_buffers()
        if chunk_bytes * self.world > self._xcap:
            return None
        idx = self._xflip
        self._xflip ^= 1
        dst = [p + self.rank * chunk_bytes for p in self._xptrs[idx]]       # my chunk of every rank's buffer
        self.C.gemm_bf16_nt_scatter(x2d, w, dst, rows)
        self.C.symm_group_barrier(self.flag_ptrs, self.expect, NUM_SLOTS - 1, NUM_SLOTS, self.rank)
        self.native.launch_counts["symm_gemm_reduce_scatter"] += 1
        return self.C.symm_sum_slots(bufs[idx], self.world, rows, N)

    def all_gather(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """Flat concatenation of every rank's ``x`` (equal sizes), or ``None`` when the tensor does
        not qualify (the caller then uses NCCL).  Each rank stores its chunk into slot ``rank`` of
        every peer's receive buffer; the context-parallel key/value gather and the sequence gathers
        of Ulysses attention take this path (the reference issues NCCL collectives there:
        chatlearn/utils/communication_op.py:30-110)."""
        return self._exchange(x.view(-1), x.numel() * x.element_size(), False)

    def all_to_all(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """Equal-split all-to-all along dim 0: chunk ``p`` of ``x`` goes to rank ``p``; the result has
        chunk ``r`` received from rank ``r``.  ``None`` when the tensor does not qualify."""
        if x.shape[0] % self.world:
            return None
        out = self._exchange(x, x.numel() * x.element_size() // self.world, True)
        return None if out is None else out.view(x.shape)

    def status(self) -> int:
        return int(self.C.symm_last_status())


_GROUPS: Dict[int, SymmGroup] = {}


def get(group: Group) -> Optional[SymmGroup]:
    """The ``SymmGroup`` of a process group (created on first use, collectively), or
    ``None`` when symmetric memory is unavailable (CPU ranks, single rank)."""
    if group is None or group.size <= 1 or group.size > 8 or not symm_mem.available():
        return None
    key = id(group.pg)
    if key not in _GROUPS:
        _GROUPS[key] = SymmGroup(group)
    return _GROUPS[key]


def attach_exchange(group: Group) -> Optional[SymmGroup]:
    """Route the group's equal-split all-gathers and all-to-alls through the peer-memory
    exchange kernels (``CLB200_SYMM_XCHG=0`` keeps NCCL).  Collective over the group."""
    if os.environ.get("CLB200_SYMM_XCHG", "1") == "0":
        return None
    sg = get(group)
    if sg is not None:
        group.fast["exchange"] = sg
    return sg


class _LinearReduceScatter(torch.autograd.Function):
    """``reduce_scatter(x @ w.T)`` along the rows, fused (forward); the backward all-gathers the output gradient
    and runs the input- and weight-gradient GEMMs of an ordinary linear layer."""

    @staticmethod
    def forward(ctx, x, w, group, sg):
        y = sg.gemm_reduce_scatter(x, w)
        ctx.save_for_backward(x, w)
        ctx.group = group
        return y

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        native = __import__("chatlearn_b200.ops.native", fromlist=["x"])
        gf = ctx.group.all_gather_cat(g.contiguous(), 0)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = native.gemm_nn(gf, w)
        if ctx.needs_input_grad[1]:
            dw = native.wgrad_accumulate(gf, x, w)
        return dx, dw, None, None


def attach_gemm_reduce_scatter(group: Group) -> Optional[SymmGroup]:
    """Route the row-parallel layers of a tensor-parallel group under sequence parallelism through the fused
    GEMM + reduce-scatter (``CLB200_SYMM_GEMM_RS=0`` keeps GEMM + NCCL).  Collective over the group."""
    if os.environ.get("CLB200_SYMM_GEMM_RS", "1") == "0":
        return None
    sg = get(group)
    if sg is None:
        return None
    world = sg.world

    def fused(x, w):
        x2 = x.reshape(-1, x.shape[-1])
        M, N = x2.shape[0], w.shape[0]
        if M == 0 or M % world or not sg.native.push_ok(x2, w) or N % 8 or (M // world) * N * 2 % 16 \
                or M * N * 2 > (int(os.environ.get("CLB200_SYMM_XCHG_MB", "192")) << 20):
            return None
        return _LinearReduceScatter.apply(x2, w, group, sg)
    group.fast["gemm_rs"] = fused
    return sg
