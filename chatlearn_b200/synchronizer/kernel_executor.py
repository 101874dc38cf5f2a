"""Runs a weight-sync plan with the descriptor-table pull kernel.

The plan's descriptors for this destination rank are compiled once into a device
table of ``{src pointer, dst pointer, strides, rows, cols}`` records.  Source
pointers are this GPU's own buffers or peer buffers mapped through symmetric
memory (``parallel.symm_mem``); the kernel reads them with plain loads over
NVLink and writes the rollout layout directly, casting on the fly.  Pointers are
re-resolved when a buffer was re-allocated (offload/onload cycles).
"""
from typing import Dict, List

import numpy as np
import torch
import torch.distributed as dist

from .plan import CopyDesc

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

_DESC = np.dtype([("src", "<u8"), ("dst", "<u8"), ("src_stride", "<i8"), ("dst_stride", "<i8"),
                  ("rows", "<i4"), ("cols", "<i4"), ("first_tile", "<i4"), ("tiles_per_row", "<i4")])


class KernelExecutor:
    def __init__(self, plan: Dict[int, List[CopyDesc]], rank: int, world: int):
        from chatlearn_b200.ops import native
        self.native = native
        assert native.C.weight_sync_desc_size() == _DESC.itemsize
        self.tile = native.C.weight_sync_tile_elems()
        self.rank, self.world = rank, world
        self.descs = self._coalesce(plan.get(rank, []))
        self.needs_peers = any(d.src_rank != rank for d in self.descs)
        self._table = None
        self._key = None
        self._total_tiles = 0

    @staticmethod
    def _coalesce(descs: List[CopyDesc]) -> List[CopyDesc]:
        """Rectangles that are contiguous on both sides become one long row."""
        out = []
        for d in descs:
            if d.rows > 1 and d.cols == d.src_stride and d.cols == d.dst_stride:
                d = CopyDesc(d.src_rank, d.src_buffer, d.src_offset, d.rows * d.cols, d.dst_rank, d.dst_buffer,
                             d.dst_offset, d.rows * d.cols, 1, d.rows * d.cols, d.hf_name)
            out.append(d)
        return out

    def _peer_ptr(self, src_bufs, name: str, src_rank: int) -> int:
        from chatlearn_b200.parallel import symm_mem
        return symm_mem.peer_pointer(src_bufs[name], src_rank)

    def _build(self, src_bufs: Dict[str, torch.Tensor], dst_bufs: Dict[str, torch.Tensor]):
        arr = np.zeros(len(self.descs), dtype=_DESC)
        tiles = 0
        sdt = ddt = None
        for i, d in enumerate(self.descs):
            dst = dst_bufs[d.dst_buffer]
            ddt = dst.dtype
            if d.src_rank == self.rank:
                src = src_bufs[d.src_buffer]
                sptr, ssz, sdt_i = src.data_ptr(), src.element_size(), src.dtype
            else:
                src = src_bufs[d.src_buffer]          # same role on every rank: same dtype
                sptr, ssz, sdt_i = self._peer_ptr(src_bufs, d.src_buffer, d.src_rank), src.element_size(), src.dtype
            assert sdt is None or sdt == sdt_i, "one source dtype per sync"
            sdt = sdt_i
            tpr = (d.cols + self.tile - 1) // self.tile
            arr[i] = (sptr + d.src_offset * ssz, dst.data_ptr() + d.dst_offset * dst.element_size(),
                      d.src_stride, d.dst_stride, d.rows, d.cols, tiles, tpr)
            tiles += tpr * d.rows
        dev = next(iter(dst_bufs.values())).device
        self._table = torch.from_numpy(arr.view(np.uint8).copy()).to(dev)
        self._total_tiles = tiles
        self._codes = (_DTYPE_CODE[sdt], _DTYPE_CODE[ddt]) if self.descs else (0, 0)

    def run(self, src_bufs: Dict[str, torch.Tensor], dst_bufs: Dict[str, torch.Tensor]):
        if self.needs_peers:
            # writers must have finished their update before anybody pulls
            dist.barrier()
        if self.descs:
            key = tuple(sorted((k, v.data_ptr()) for k, v in list(src_bufs.items()) + list(dst_bufs.items())))
            if key != self._key:
                self._build(src_bufs, dst_bufs)
                self._key = key
            self.native.weight_sync_run(self._table, len(self.descs), self._total_tiles, *self._codes)
        if self.needs_peers:
            # nobody may overwrite its source while a peer is still reading it
            torch.cuda.current_stream().synchronize()
            dist.barrier()
