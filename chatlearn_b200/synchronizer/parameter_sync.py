"""Parameter synchronisation trainer → rollout.

Parity: chatlearn/synchronizer/parameter_sync.py:53-239 (initialise: collect
metadata, map, validate, plan; ``sync()`` = pre → transfer → post) and
chatlearn/synchronizer/parameter_sync_fsdp.py:27-57 (FSDP path).  One class
serves both trainer back ends because both publish the same rectangle layout.

Execution back ends, chosen per call:

* ``kernel``  – every destination GPU runs one descriptor-table kernel that pulls
  its rectangles from peer (or its own) memory with the cast fused in; needs the
  source buffers in symmetric memory (CUDA only);
* ``p2p``     – portable path: per (sender, receiver) pair the sender packs its
  pieces (already cast) into one message, ``batch_isend_irecv`` moves it, the
  receiver unpacks; this is also the NCCL baseline the kernel is compared with;
* local-only plans (every rectangle already on the destination rank) run as
  strided copies with no communication in either mode.
"""
import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from chatlearn_b200.utils.logger import logger
from .plan import BufferInfo, CopyDesc, LeafPlacement, RankLayout, build_plan, plan_stats, validate_plan


def layout_of_model(model, rank: int, shard_of_block=None, prefix: str = "") -> RankLayout:
    """Publish a ``CausalLM``'s blocks.  ``shard_of_block(name) -> (lo, hi) | None``
    tells which element range of each block this rank actually holds."""
    lay = RankLayout(rank)
    for b in model.blocks:
        shard = shard_of_block(b.name) if shard_of_block else None
        lay.buffers[prefix + b.name] = BufferInfo(prefix + b.name, b.numel, str(b.dtype), shard)
        for lf in b.leaves:
            lay.leaves.append(LeafPlacement(lf, prefix + b.name, b.offsets[lf.name]))
    return lay


def _view2d(buf: torch.Tensor, offset: int, stride: int, rows: int, cols: int) -> torch.Tensor:
    # as_strided takes an offset into the *storage*: a buffer that is itself a slice of a larger allocation
    # (the parameter slices of a sharded trainer live in one arena) starts at its own storage offset
    return torch.as_strided(buf, (rows, cols), (stride, 1), buf.storage_offset() + offset)


class ParameterSyncGroup:
    def __init__(self, src_model, dst_model, world_group=None, mode: str = "auto"):
        """``src_model`` / ``dst_model`` are modules exposing ``sync_layout()`` →
        ``RankLayout`` (or ``None`` on ranks that do not host the role) and
        ``sync_buffers()`` → ``{buffer name: flat tensor}``."""
        self.src, self.dst = src_model, dst_model
        self.group = world_group
        self.mode = mode
        self.plan: Optional[Dict[int, List[CopyDesc]]] = None
        self.stats: Dict[str, float] = {}
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self._kernel_state = None
        self.last_ms = 0.0

    # ------------------------------------------------------------------ planning
    def initialize(self):
        src_lay = self.src.sync_layout() if self.src.is_member else None
        dst_lay = self.dst.sync_layout() if self.dst.is_member else None
        if self.world > 1:
            gathered = [None] * self.world
            dist.all_gather_object(gathered, (src_lay, dst_lay))
        else:
            gathered = [(src_lay, dst_lay)]
        src_layouts = [g[0] for g in gathered if g[0] is not None]
        dst_layouts = [g[1] for g in gathered if g[1] is not None]
        assert src_layouts and dst_layouts, "parameter sync needs a source and a destination"
        t0 = time.perf_counter()
        self.plan = build_plan(src_layouts, dst_layouts)
        validate_plan(self.plan, dst_layouts)
        esz = 2
        self.stats = plan_stats(self.plan, esz)
        self.stats["plan_s"] = time.perf_counter() - t0
        if self.rank == 0:
            logger.info(f"parameter sync {self.src.name}->{self.dst.name}: {self.stats}")
        return self

    # ------------------------------------------------------------------ execution
    def _all_local(self) -> bool:
        return all(d.src_rank == dst for dst, ds in self.plan.items() for d in ds)

    @torch.no_grad()
    def _run_local(self, descs: List[CopyDesc], src_bufs, dst_bufs):
        for d in descs:
            s = _view2d(src_bufs[d.src_buffer], d.src_offset, d.src_stride, d.rows, d.cols)
            t = _view2d(dst_bufs[d.dst_buffer], d.dst_offset, d.dst_stride, d.rows, d.cols)
            t.copy_(s)

    @torch.no_grad()
    def _run_p2p(self, src_bufs, dst_bufs):
        me = self.rank
        mine = self.plan.get(me, [])
        self._run_local([d for d in mine if d.src_rank == me], src_bufs, dst_bufs)
        # what I send: pieces of every destination whose source is me
        send: Dict[int, List[CopyDesc]] = {}
        for dst, ds in self.plan.items():
            if dst == me:
                continue
            for d in ds:
                if d.src_rank == me:
                    send.setdefault(dst, []).append(d)
        recv: Dict[int, List[CopyDesc]] = {}
        for d in mine:
            if d.src_rank != me:
                recv.setdefault(d.src_rank, []).append(d)
        if not send and not recv:
            return
        dst_dtype = None
        if dst_bufs:
            dst_dtype = next(iter(dst_bufs.values())).dtype
        dev = next(iter((src_bufs or dst_bufs).values())).device
        ops_, keep = [], []
        # the message dtype is the destination dtype: the cast happens at the source
        wire = self._wire_dtype(dst_dtype, dev)
        for dst, ds in sorted(send.items()):
            msg = torch.empty(sum(d.numel for d in ds), dtype=wire, device=dev)
            off = 0
            for d in ds:
                s = _view2d(src_bufs[d.src_buffer], d.src_offset, d.src_stride, d.rows, d.cols)
                msg[off:off + d.numel].view(d.rows, d.cols).copy_(s)
                off += d.numel
            keep.append(msg)
            ops_.append(dist.P2POp(dist.isend, msg, dst))
        inbox = {}
        for src, ds in sorted(recv.items()):
            msg = torch.empty(sum(d.numel for d in ds), dtype=wire, device=dev)
            inbox[src] = msg
            ops_.append(dist.P2POp(dist.irecv, msg, src))
        if ops_:
            for req in dist.batch_isend_irecv(ops_):
                req.wait()
        for src, ds in recv.items():
            msg, off = inbox[src], 0
            for d in ds:
                t = _view2d(dst_bufs[d.dst_buffer], d.dst_offset, d.dst_stride, d.rows, d.cols)
                t.copy_(msg[off:off + d.numel].view(d.rows, d.cols))
                off += d.numel

    def _wire_dtype(self, dst_dtype, dev):
        """All ranks must agree on the message dtype even if they host one side only."""
        code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
        inv = {v: k for k, v in code.items()}
        t = torch.tensor([code.get(dst_dtype, -1)], device=dev if dev.type == "cuda" else "cpu")
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return inv[int(t.item())]

    @torch.no_grad()
    def sync(self):
        """Run one synchronisation; returns elapsed milliseconds on this rank."""
        if self.plan is None:
            self.initialize()
        self.src.pre_parameter_sync()
        self.dst.pre_parameter_sync()
        src_bufs = self.src.sync_buffers() if self.src.is_member else {}
        dst_bufs = self.dst.sync_buffers() if self.dst.is_member else {}
        cuda = any(t.is_cuda for t in list(src_bufs.values()) + list(dst_bufs.values()))
        if cuda:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        t0 = time.perf_counter()
        mode = self.mode
        if mode == "auto":
            mode = "kernel" if cuda else "p2p"
        if mode == "kernel":
            from .kernel_executor import KernelExecutor
            if self._kernel_state is None:
                self._kernel_state = KernelExecutor(self.plan, self.rank, self.world)
            self._kernel_state.run(src_bufs, dst_bufs)
        elif self._all_local():
            self._run_local(self.plan.get(self.rank, []), src_bufs, dst_bufs)
        else:
            self._run_p2p(src_bufs, dst_bufs)
        if cuda:
            ev1.record()
            ev1.synchronize()
            self.last_ms = ev0.elapsed_time(ev1)
        else:
            self.last_ms = (time.perf_counter() - t0) * 1e3
        self.src.post_parameter_sync()
        self.dst.post_parameter_sync()
        return self.last_ms
