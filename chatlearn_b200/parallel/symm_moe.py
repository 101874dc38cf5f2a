"""Expert-parallel MoE layer without all-to-all: dispatch and combine through peer memory.

The NCCL path of ``ExpertParallel.experts`` exchanges per-expert counts, then the tokens, runs
the experts, and sends the results back (four collectives per layer, the role of Megatron's
``alltoall`` token dispatcher in the reference, chatlearn/utils/megatron_utils.py:61).  Here
every rank owns symmetric receive buffers with a fixed-capacity region per local expert; the
dispatch kernel claims rows with remote atomics and stores tokens straight into the owner's
region, the grouped tcgen05 GEMM runs over the occupied part of the regions (tile table built
on the device from the row cursors), and the combine kernel pulls the outputs back.  Used for
inference (rollout); training keeps the differentiable NCCL path.

Capacity: ``capacity_factor`` × the mean rows per expert for the largest step seen so far
(buffers grow collectively when a larger step arrives).  A full region drops the pair and sets
status 2, which ``status()`` reports; the rollout engine checks it after every ``generate`` call and
raises (an overflow means the capacity factor is too small for the routing skew: the outputs of that
call are not used).
"""
from typing import Optional

import torch

from . import symm_mem
from .groups import Group

NUM_SLOTS = 64


class SymmMoE:
    def __init__(self, group: Group, num_experts: int, hidden: int, capacity_factor: float = 4.0):
        from chatlearn_b200.ops import native
        self.C, self.native = native.C, native
        self.group, self.pg = group, group.pg
        self.rank, self.world = group.rank, group.size
        assert 1 < self.world <= 8 and num_experts % self.world == 0
        self.E, self.El, self.H = num_experts, num_experts // self.world, hidden
        self.factor = capacity_factor
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.flags = symm_mem.empty(8 * NUM_SLOTS, torch.int32, self.device, group=self.pg)
        self.flags.zero_()
        self.expect = torch.zeros(NUM_SLOTS * 8, dtype=torch.int32, device=self.device)
        self.flag_ptrs = self._ptrs(self.flags)
        self.cursor = symm_mem.empty(max(self.El, 4), torch.int32, self.device, group=self.pg)
        self.cursor.zero_()
        self.cursor_ptrs = self._ptrs(self.cursor)
        self.cap = 0
        self._slot = 0
        torch.cuda.synchronize()
        group.barrier()

    def _ptrs(self, t):
        return [symm_mem.peer_pointer(t, self.group.ranks[r]) for r in range(self.world)]

    def _barrier(self):
        self.C.symm_moe_barrier(self.flag_ptrs, self.expect, self._slot, NUM_SLOTS, self.rank)
        self._slot = (self._slot + 1) % NUM_SLOTS

    def _ensure_capacity(self, pairs_per_rank: int):
        """Collective: every rank passes the same value (the largest per-rank step size)."""
        need = int(self.factor * pairs_per_rank * self.world / self.E) + 128
        need = (need + 127) // 128 * 128
        if need <= self.cap:
            return
        self.cap = need
        rows = self.El * self.cap
        self.recv_x = symm_mem.empty(rows * self.H, torch.bfloat16, self.device, group=self.pg)
        self.recv_y = symm_mem.empty(rows * self.H, torch.bfloat16, self.device, group=self.pg)
        self.recv_x_ptrs, self.recv_y_ptrs = self._ptrs(self.recv_x), self._ptrs(self.recv_y)
        self._h13 = self._act = None                      # expert intermediates, sized on first use
        torch.cuda.synchronize()
        self.group.barrier()

    @torch.no_grad()
    def experts(self, x, w13, w2, weights, idx, pairs_per_rank: Optional[int] = None):
        """``x [T, H]`` bf16; ``w13 [El, 2F, H]``, ``w2 [El, H, F]`` are this rank's experts; ``idx``
        holds global expert ids.  ``pairs_per_rank``: upper bound of T·k over the ranks (defaults to
        this rank's, which is right when all ranks carry the same number of tokens)."""
        T, k = idx.shape
        self._ensure_capacity(pairs_per_rank if pairs_per_rank is not None else T * k)
        rows = self.El * self.cap
        self._barrier()                                   # cursors are zero and the buffers free everywhere
        where = self.C.symm_moe_dispatch(x.contiguous(), idx.contiguous(), self.recv_x_ptrs, self.cursor_ptrs, self.El, self.cap)
        self._barrier()                                   # every rank's tokens have landed
        xs = self.recv_x.view(rows, self.H)
        F2 = w13.shape[1]
        table, count = self.C.symm_moe_region_table(self.cursor[:self.El], self.cap, F2)
        if self._h13 is None or self._h13.shape != (rows, F2):
            self._h13 = torch.empty(rows, F2, dtype=torch.bfloat16, device=self.device)
            self._act = torch.empty(rows, F2 // 2, dtype=torch.bfloat16, device=self.device)
        self.C.grouped_gemm_bf16_nt_table(xs, w13, table, count, self._h13)
        self.C.symm_moe_swiglu(self._h13, self._act, table, count)         # occupied rows only
        table2, count2 = self.C.symm_moe_region_table(self.cursor[:self.El], self.cap, w2.shape[1])
        self.C.grouped_gemm_bf16_nt_table(self._act, w2, table2, count2, self.recv_y.view(rows, self.H))
        self._barrier()                                   # every rank's expert outputs are written
        out = self.C.symm_moe_combine(self.recv_y_ptrs, where, weights.float(), self.H, rows)
        self._barrier()                                   # nobody still reads my outputs ...
        self.cursor.zero_()                               # ... before the regions are handed out again
        for name, n in (("symm_moe_dispatch", 1), ("grouped_gemm_bf16_nt", 2), ("swiglu_fwd", 1), ("symm_moe_combine", 1)):
            self.native.launch_counts[name] += n
        return out

    def status(self) -> int:
        return int(self.C.symm_moe_last_status())
