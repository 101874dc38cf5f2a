"""Packed (varlen) attention on this package's forward kernel.

``csrc/attention_fwd.cu`` covers every pass that needs no gradient: prompt prefill in
the rollout engine and the behaviour / reference log-prob forwards.  A pass that will be
differentiated goes to the library statement (flash-attn forward + backward), as the
reference does for all of them (chatlearn/models/fsdp_module.py:257,269
``attn_implementation="flash_attention_2"``).  ``CLB200_ATTN=library`` forces the library
for every pass.
"""
import math
import os

import torch

from . import library_counts, reference as ref, register_native
from . import native as _n

C = _n.C
_FORCE_LIBRARY = os.environ.get("CLB200_ATTN", "native") == "library"
# head dim 128: "tcgen05" (tensor-memory kernel, csrc/attention_sm100.cu) or "mma" (the warp-level MMA kernel that
# also serves head dim 64)
_IMPL = os.environ.get("CLB200_ATTN_FWD", "tcgen05")


def set_fwd_impl(name: str):
    global _IMPL
    assert name in ("tcgen05", "mma")
    _IMPL = name


def _ok(x, D):
    return (x.dim() == 3 and x.dtype == torch.bfloat16 and x.shape[2] == D and x.stride(2) == 1 and x.stride(1) == D
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)


def attention_varlen(q, k, v, cu_seqlens, max_seqlen=None, scale=None, causal=True):
    D = q.shape[-1]
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if (_FORCE_LIBRARY or needs_grad or D not in (64, 128) or v.shape[-1] != D
            or not (_ok(q, D) and _ok(k, D) and _ok(v, D)) or q.shape[1] % k.shape[1] != 0):
        library_counts["attention_varlen"] += 1
        return ref.attention_varlen(q, k, v, cu_seqlens, max_seqlen, scale, causal)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    cu = cu_seqlens if cu_seqlens.dtype == torch.int32 else cu_seqlens.to(torch.int32)
    if D == 128 and _IMPL == "tcgen05":
        out, _lse = C.attn_fwd_sm100(q, k, v, cu.contiguous(), float(scale), bool(causal))
    else:
        out, _lse = C.attn_varlen_fwd(q, k, v, cu.contiguous(), float(scale), bool(causal))
    _n._count("attn_varlen_fwd")
    return out


register_native("attention_varlen", attention_varlen)
