"""Host <-> device transfers with byte accounting.

Step inputs (token ids, positions, slot maps, packed training rows) are staged in
pinned host memory and copied asynchronously; results read back (sampled ids, loss
statistics) are counted too.  The counters let the benchmark report how many
bytes cross PCIe per step."""
from typing import Dict

import torch

h2d_bytes = 0
d2h_bytes = 0
_pinned: Dict[tuple, torch.Tensor] = {}


def reset():
    global h2d_bytes, d2h_bytes
    h2d_bytes = d2h_bytes = 0


def to_device(t: torch.Tensor, device, slot: str = "") -> torch.Tensor:
    """Copy a CPU tensor to ``device`` through a pinned staging buffer."""
    global h2d_bytes
    device = torch.device(device)
    if device.type != "cuda" or t.device.type != "cpu":
        return t.to(device)
    n = t.numel()
    h2d_bytes += n * t.element_size()
    if n == 0:
        return torch.empty(t.shape, dtype=t.dtype, device=device)
    if not t.is_pinned():
        key = (slot, t.dtype)
        buf = _pinned.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1024), dtype=t.dtype, pin_memory=True)
            _pinned[key] = buf
        # the staging buffer is reused: make sure the previous copy out of it is done
        ev = getattr(buf, "_ev", None)
        if ev is not None:
            ev.synchronize()
        stage = buf[:n].view(t.shape) if t.is_contiguous() else buf[:n].view(t.shape)
        stage.copy_(t)
        out = stage.to(device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        buf._ev = ev
        return out
    return t.to(device, non_blocking=True)


def to_host(t: torch.Tensor) -> torch.Tensor:
    global d2h_bytes
    if t.device.type == "cuda":
        d2h_bytes += t.numel() * t.element_size()
    return t.cpu()


def tolist(t: torch.Tensor):
    return to_host(t).tolist()


def item(t: torch.Tensor):
    return to_host(t).item()
