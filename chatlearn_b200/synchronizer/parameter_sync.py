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
  receiver unpacks; this is also the NCCL baseline the kernel is compared with.
  The transfer runs in iterations planned under a memory budget (``plan.build_iterations``:
  messages of at most ``bucket_size_mb``, and per iteration no rank stages more than
  ``max_memory_fraction`` of its device memory minus what is already in use);
* local-only plans (every rectangle already on the destination rank) run as
  strided copies with no communication in either mode.
"""
import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from chatlearn_b200.utils.logger import logger
from .plan import (BufferInfo, CopyDesc, LeafPlacement, RankLayout, build_iterations, build_plan, iteration_stats,
                   plan_stats, validate_plan)


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
    def __init__(self, src_model, dst_model, world_group=None, mode: str = "auto", bucket_size_mb: float = 1024,
                 max_memory_fraction: float = 0.8):
        """``src_model`` / ``dst_model`` are modules exposing ``sync_layout()`` →
        ``RankLayout`` (or ``None`` on ranks that do not host the role) and
        ``sync_buffers()`` → ``{buffer name: flat tensor}``."""
        self.src, self.dst = src_model, dst_model
        self.group = world_group
        self.mode = mode
        self.bucket_bytes = max(int(float(bucket_size_mb) * (1 << 20)), 1024)
        self.max_memory_fraction = float(max_memory_fraction)
        self.iterations = None
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

    def _staging_budgets(self, dev) -> Dict[int, int]:
        """Bytes every rank may stage per iteration: ``max_memory_fraction`` of its device memory minus what is in
        use now (chatlearn/synchronizer/planners/tensor_planner.py:100-108).  CPU ranks are not bounded."""
        mine = -1
        if dev.type == "cuda":
            free, total = torch.cuda.mem_get_info(dev)
            # memory this process has cached but not allocated can be reused for the messages
            free += torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)
            mine = int(free - (1.0 - self.max_memory_fraction) * total)
        got = [mine]
        if self.world > 1:
            got = [None] * self.world
            dist.all_gather_object(got, mine)
        return {r: max(b, 1 << 20) for r, b in enumerate(got) if b is not None and b >= 0}

    def _plan_iterations(self, dev, elem_size: int):
        if self.iterations is None:
            self.iterations = build_iterations(self.plan, elem_size, self.bucket_bytes, self._staging_budgets(dev))
            self.stats.update(iteration_stats(self.iterations, elem_size))
            if self.rank == 0:
                logger.info(f"parameter sync {self.src.name}->{self.dst.name}: {self.stats['iterations']} iteration(s), "
                            f"at most {self.stats['peak_staged_mb']} MB staged per rank")
        return self.iterations

    @torch.no_grad()
    def _run_p2p(self, src_bufs, dst_bufs):
        me = self.rank
        mine = self.plan.get(me, [])
        self._run_local([d for d in mine if d.src_rank == me], src_bufs, dst_bufs)
        if all(d.src_rank == dst for dst, ds in self.plan.items() for d in ds):
            return
        dst_dtype = None
        if dst_bufs:
            dst_dtype = next(iter(dst_bufs.values())).dtype
        bufs = src_bufs or dst_bufs
        dev = next(iter(bufs.values())).device if bufs else \
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        # the message dtype is the destination dtype: the cast happens at the source
        wire = self._wire_dtype(dst_dtype, dev)
        for it in self._plan_iterations(dev, torch.empty(0, dtype=wire).element_size()):
            send = {dst: ds for (src, dst), ds in it.items() if src == me}
            recv = {src: ds for (src, dst), ds in it.items() if dst == me}
            if send or recv:
                self._exchange(send, recv, src_bufs, dst_bufs, wire, dev)

    def _exchange(self, send, recv, src_bufs, dst_bufs, wire, dev):
        ops_, keep = [], []
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
