"""Residency management: moving flat device buffers to pinned host memory and back.

Parity: chatlearn/utils/flat_tensors.py:44-287 (``FlatTensors`` /
``BucketizedFlatTensors``: aggregate tensors in one buffer, pinned CPU primary
store, async D2H/H2D) and the Megatron memory managers
(chatlearn/models/megatron/memory_manager/trainer.py:173-442).  Parameters here
already live in one flat buffer per block, so offload is one large DMA per block
on a dedicated copy stream into a pre-pinned host arena; the arena is allocated
once and reused every episode (no ``cudaHostRegister`` per call, no pageable
``model.cpu()`` as in chatlearn/models/fsdp_module.py:543-575).
"""
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch


class FlatTensors:
    """A set of tensors aggregated in one flat device buffer with a host copy.

    ``tensors`` are re-pointed (``t.data``) at views of the flat buffer.  After
    ``copy_to_primary_store`` the device buffer is released and the tensors hold
    empty storage; ``copy_to_gpu_buffer`` restores them."""

    def __init__(self, tensors: Sequence[torch.Tensor], primary_store_device="cpu",
                 pin: bool = True):
        self._tensors = list(tensors)
        self._shapes = [t.shape for t in self._tensors]
        self._numels = [t.numel() for t in self._tensors]
        self.total_numel = sum(self._numels)
        self._dtype = self._tensors[0].dtype if self._tensors else torch.float32
        assert all(t.dtype == self._dtype for t in self._tensors), "one dtype per FlatTensors"
        self._device = self._tensors[0].device if self._tensors else torch.device("cpu")
        self._pin = pin and torch.cuda.is_available()
        self._primary: Optional[torch.Tensor] = None
        self._gpu: Optional[torch.Tensor] = None
        self._stream = torch.cuda.Stream() if self._device.type == "cuda" else None
        self._aggregate()

    def _aggregate(self):
        buf = torch.empty(self.total_numel, dtype=self._dtype, device=self._device)
        off = 0
        for t, n, shp in zip(self._tensors, self._numels, self._shapes):
            buf[off:off + n].copy_(t.detach().reshape(-1))
            t.data = buf[off:off + n].view(shp)
            off += n
        self._gpu = buf

    @property
    def in_gpu(self) -> bool:
        return self._gpu is not None

    def _host(self) -> torch.Tensor:
        if self._primary is None:
            self._primary = torch.empty(self.total_numel, dtype=self._dtype, device="cpu",
                                        pin_memory=self._pin)
        return self._primary

    @torch.no_grad()
    def copy_to_primary_store(self, non_blocking: bool = True):
        if self._gpu is None:
            return
        host = self._host()
        if self._stream is not None:
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                host.copy_(self._gpu, non_blocking=non_blocking)
            self._gpu.record_stream(self._stream)
            self._stream.synchronize()
        else:
            host.copy_(self._gpu)
        for t in self._tensors:
            t.data = torch.empty(0, dtype=self._dtype, device=self._device)
        self._gpu = None

    @torch.no_grad()
    def copy_to_gpu_buffer(self, non_blocking: bool = True):
        if self._gpu is not None:
            return
        buf = torch.empty(self.total_numel, dtype=self._dtype, device=self._device)
        if self._stream is not None:
            with torch.cuda.stream(self._stream):
                buf.copy_(self._host(), non_blocking=non_blocking)
            torch.cuda.current_stream().wait_stream(self._stream)
        else:
            buf.copy_(self._host())
        off = 0
        for t, n, shp in zip(self._tensors, self._numels, self._shapes):
            t.data = buf[off:off + n].view(shp)
            off += n
        self._gpu = buf

    def release_gpu_buffer(self):
        for t in self._tensors:
            t.data = torch.empty(0, dtype=self._dtype, device=self._device)
        self._gpu = None


class BucketizedFlatTensors:
    """``FlatTensors`` split into buckets of at most ``bucket_size_mb``."""

    def __init__(self, tensors: Sequence[torch.Tensor], bucket_size_mb: int = 1024,
                 primary_store_device="cpu"):
        limit = bucket_size_mb * (1 << 20)
        buckets: List[List[torch.Tensor]] = []
        cur, cur_bytes, cur_dtype = [], 0, None
        for t in tensors:
            nbytes = t.numel() * t.element_size()
            if cur and (cur_bytes + nbytes > limit or t.dtype != cur_dtype):
                buckets.append(cur)
                cur, cur_bytes = [], 0
            cur.append(t)
            cur_bytes += nbytes
            cur_dtype = t.dtype
        if cur:
            buckets.append(cur)
        self._flat = [FlatTensors(b, primary_store_device) for b in buckets]

    def copy_to_primary_store(self, non_blocking=True):
        for f in self._flat:
            f.copy_to_primary_store(non_blocking)

    def copy_to_gpu_buffer(self, non_blocking=True):
        for f in self._flat:
            f.copy_to_gpu_buffer(non_blocking)

    def release_gpu_buffer(self):
        for f in self._flat:
            f.release_gpu_buffer()

    @property
    def in_gpu(self):
        return all(f.in_gpu for f in self._flat)


class ResidencyManager:
    """Offload / onload of attribute-held flat tensors by tag.

    ``items`` are ``(owner, attr)`` pairs whose value is a flat tensor; an optional
    ``rebind(owner, tensor)`` callback re-points dependent views after onload
    (parameter blocks re-bind their leaves).  Host arenas are pinned and cached
    per (owner, attr); copies run on one copy stream and are fenced to the
    compute stream with events, so an offload overlaps whatever the compute
    stream does next and an onload overlaps what it did before."""

    def __init__(self, device, pin: bool = True):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.pin = pin and self.cuda
        self.stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self._host: Dict[Tuple[int, str], torch.Tensor] = {}
        self._meta: Dict[Tuple[int, str], Tuple[torch.dtype, int]] = {}
        self.bytes_offloaded = 0

    def _arena(self, key, t: torch.Tensor) -> torch.Tensor:
        h = self._host.get(key)
        if h is None or h.numel() != t.numel() or h.dtype != t.dtype:
            h = torch.empty(t.numel(), dtype=t.dtype, device="cpu", pin_memory=self.pin)
            self._host[key] = h
        return h

    @torch.no_grad()
    def offload(self, items, release: Optional[Callable] = None, unchanged: bool = False):
        """``unchanged=True``: the device tensors were not modified since they were
        last onloaded (frozen models), so an existing host copy is still valid and
        the device copy is simply dropped."""
        pending = []
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
        for owner, attr in items:
            t = getattr(owner, attr, None)
            if t is None or t.device.type == "cpu" or t.numel() == 0:
                continue
            key = (id(owner), attr)
            if unchanged and key in self._meta and key in self._host \
                    and self._host[key].numel() == t.numel():
                pending.append((owner, attr))
                continue
            h = self._arena(key, t)
            self._meta[key] = (t.dtype, t.numel())
            if self.cuda:
                with torch.cuda.stream(self.stream):
                    h.copy_(t.reshape(-1), non_blocking=True)
                t.record_stream(self.stream)
            else:
                h.copy_(t.reshape(-1))
            self.bytes_offloaded += t.numel() * t.element_size()
            pending.append((owner, attr))
        if self.cuda:
            self.stream.synchronize()
        for owner, attr in pending:
            if release is not None:
                release(owner, attr)
            else:
                setattr(owner, attr, None)

    @torch.no_grad()
    def onload(self, items, rebind: Optional[Callable] = None):
        for owner, attr in items:
            key = (id(owner), attr)
            if key not in self._meta:
                continue
            cur = getattr(owner, attr, None)
            if cur is not None and cur.numel() > 0 and cur.device.type != "cpu":
                continue
            dtype, n = self._meta[key]
            t = torch.empty(n, dtype=dtype, device=self.device)
            if self.cuda:
                with torch.cuda.stream(self.stream):
                    t.copy_(self._host[key], non_blocking=True)
            else:
                t.copy_(self._host[key])
            if rebind is not None:
                rebind(owner, attr, t)
            else:
                setattr(owner, attr, t)
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
