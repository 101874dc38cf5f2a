"""Packed (varlen) attention on this package's kernels.

Head dim 128 runs on the tensor-memory kernels: ``csrc/attention_sm100.cu`` (forward, with the
log-sum-exp kept for the backward) and ``csrc/attention_bwd_sm100.cu`` (dQ, dK, dV), for passes
with and without a gradient: prompt prefill in the rollout engine, the behaviour / reference
log-prob forwards and the trainer's forward + backward.  Head dim 64 has the warp-level MMA
forward of ``csrc/attention_fwd.cu`` for passes without a gradient; what no kernel covers (other
head dims, a gradient at head dim 64) goes to the library statement, which is what the reference
uses for every pass (chatlearn/models/fsdp_module.py:257,269
``attn_implementation="flash_attention_2"``), and is counted in ``ops.library_counts``.
``CLB200_ATTN=library`` forces the library for every pass.
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


class _AttnVarlen128(torch.autograd.Function):
    """Forward and backward of packed attention at head dim 128 on the tensor-memory kernels."""

    @staticmethod
    def forward(ctx, q, k, v, cu, scale, causal):
        out, lse = C.attn_fwd_sm100(q, k, v, cu, scale, causal)
        _n._count("attn_varlen_fwd")
        ctx.save_for_backward(q, k, v, out, lse, cu)
        ctx.scale, ctx.causal = scale, causal
        return out

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, out, lse, cu = ctx.saved_tensors
        if not _ok(d_out, 128):
            d_out = d_out.contiguous()
        dq, dk, dv = C.attn_bwd_sm100(q, k, v, out, d_out, lse, cu, ctx.scale, ctx.causal)
        _n._count("attn_varlen_bwd", 3)
        return dq, dk, dv, None, None, None


def attention_varlen(q, k, v, cu_seqlens, max_seqlen=None, scale=None, causal=True):
    D = q.shape[-1]
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    shapes_ok = (D in (64, 128) and v.shape[-1] == D and _ok(q, D) and _ok(k, D) and _ok(v, D)
                 and q.shape[1] % k.shape[1] == 0)
    if needs_grad and shapes_ok and D == 128 and _IMPL == "tcgen05" and not _FORCE_LIBRARY:
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
        cu = cu_seqlens if cu_seqlens.dtype == torch.int32 else cu_seqlens.to(torch.int32)
        return _AttnVarlen128.apply(q, k, v, cu.contiguous(), float(scale), bool(causal))
    if _FORCE_LIBRARY or needs_grad or not shapes_ok:
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
