"""Symmetric memory: buffers every rank of a group can address directly.

Fused compute+communication kernels read or write peer GPU memory with ordinary
loads/stores over NVLink; for that each rank needs the device addresses of its
peers' buffers.  Allocation and handle exchange use
``torch.distributed._symmetric_memory`` (CUDA VMM allocation + fabric/fd handle
exchange); the kernels that use the pointers are this package's own.  On CPU
ranks (gloo) nothing is allocated and ``available()`` is False.

Only plain peer loads and stores are used on these buffers: no kernel here issues
``multimem`` instructions, so binding the allocations to an NVLink multicast object
would buy nothing, and a rank that dies while its memory is bound to one can raise
NVLink faults on the surviving ranks' GPUs.  ``TORCH_SYMM_MEM_DISABLE_MULTICAST=1`` is
therefore set (unless the caller chose otherwise) before the first allocation.
"""
import os
from typing import Dict, List

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

import torch
import torch.distributed as dist

_REG: Dict[int, dict] = {}      # storage data_ptr -> {"handle", "base", "group"}


def available() -> bool:
    if not (torch.cuda.is_available() and dist.is_initialized()):
        return False
    try:
        import importlib
        importlib.import_module("torch.distributed._symmetric_memory")
        return True
    except Exception:
        return False


def empty(numel: int, dtype, device, group=None) -> torch.Tensor:
    """Allocate ``numel`` elements of symmetric memory and exchange handles
    (collective over ``group``)."""
    import torch.distributed._symmetric_memory as sm
    group = group or dist.group.WORLD
    t = sm.empty(numel, dtype=dtype, device=device)
    h = sm.rendezvous(t, group=group.group_name if hasattr(group, "group_name") else group)
    _REG[t.data_ptr()] = {"handle": h, "base": t.data_ptr(), "numel": numel, "esz": t.element_size(),
                          "group": group}
    return t


def _find(t: torch.Tensor):
    p = t.data_ptr()
    for base, rec in _REG.items():
        if base <= p < base + rec["numel"] * rec["esz"]:
            return rec, p - base
    return None, 0


def is_symmetric(t: torch.Tensor) -> bool:
    return _find(t)[0] is not None


def peer_pointer(t: torch.Tensor, global_rank: int) -> int:
    """Device address, on this GPU, of the peer's copy of ``t`` (same offset in the
    peer's symmetric allocation)."""
    rec, off = _find(t)
    if rec is None:
        raise RuntimeError("tensor is not in symmetric memory; allocate it with symm_mem.empty()")
    grank = dist.get_group_rank(rec["group"], global_rank) if rec["group"] is not dist.group.WORLD else global_rank
    return int(rec["handle"].buffer_ptrs[grank]) + off


def signal_pad_pointers(t: torch.Tensor) -> List[int]:
    rec, _ = _find(t)
    return [int(p) for p in rec["handle"].signal_pad_ptrs]
