"""Bindings of the hand-written sm_100a kernels to the op facade.

Importing this module loads ``chatlearn_b200/_C.so`` (built in-tree by
``chatlearn_b200.csrc.build``) and registers one implementation per op.  A
missing or unloadable extension raises here: on a GPU box the CUDA path must be
the one that runs.  Ops whose shapes a kernel does not cover fall back to the
PyTorch statement *for that call* and are counted in ``ops.library_counts``.
"""
import importlib.util
import math
import os

import torch

from . import launch_counts, library_counts, reference as ref, register_native

_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C.so")


def _fresh_binary():
    """The shared object must match the sources beside it: a hash of ``csrc/`` is baked into it at
    build time.  A missing or stale binary is rebuilt in place when a compiler is at hand (one
    builder at a time, the other ranks wait on a file lock); otherwise the import fails with one
    line that says so, instead of an AttributeError on a missing kernel later."""
    from chatlearn_b200.csrc import build as _b
    want, have = _b.source_hash(), _b.binary_hash(_SO)
    if have == want:
        return
    why = f"{_SO} is {'missing' if have is None and not os.path.exists(_SO) else 'stale'} " \
          f"(built from sources {have}, sources here are {want})"
    import shutil
    if os.environ.get("CLB200_NO_REBUILD") == "1" or shutil.which("nvcc") is None:
        raise ImportError(why + ": run `python -m chatlearn_b200.csrc.build` "
                          "(CUDA tensors need the sm_100a extension; there is no silent fallback)")
    import warnings
    warnings.warn(why + ": rebuilding")
    _b.build()
    if _b.binary_hash(_SO) != want:
        raise ImportError(why + " and the rebuild did not produce a matching binary")


_fresh_binary()
_spec = importlib.util.spec_from_file_location("chatlearn_b200._C", _SO)
C = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(C)

# which GEMM the linear layers use on CUDA: "tcgen05" (own kernel) or "cublas"
_GEMM_IMPL = os.environ.get("CHATLEARN_GEMM", "tcgen05")


def set_gemm_impl(name: str):
    global _GEMM_IMPL
    assert name in ("tcgen05", "cublas")
    _GEMM_IMPL = name


def get_gemm_impl():
    return _GEMM_IMPL


def _count(name, n=1):
    launch_counts[name] += n


# ------------------------------------------------------------------ rmsnorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        xc = x.contiguous()
        y, rstd = C.rmsnorm_fwd(xc, w.contiguous(), eps)
        _count("rmsnorm_fwd")
        ctx.save_for_backward(xc, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dx, dw = C.rmsnorm_bwd(x, w.contiguous(), dy.contiguous(), rstd)
        _count("rmsnorm_bwd")
        return dx, dw.to(w.dtype), None


def rmsnorm(x, w, eps):
    if x.dtype not in (torch.float32, torch.bfloat16) or w.dtype != x.dtype \
            or x.shape[-1] % (16 // x.element_size()) != 0:
        library_counts["rmsnorm"] += 1
        return ref.rmsnorm(x, w, eps)
    return _RMSNorm.apply(x, w, eps)


class SplitKPlanes:
    """Result of a K-sliced GEMM whose fp32 partial planes have not been added up yet.  ``planes`` [S, M, N] is a
    view of the per-device split-K workspace: it is valid until the next K-sliced GEMM on the device, so the
    consumer (``add_rmsnorm_`` or ``qkv_rope_append``, which add the planes up while they do their own work) must be
    the next kernel.  ``shape`` / ``out`` describe the bf16 result that was not written."""
    __slots__ = ("out", "planes")

    def __init__(self, out, planes):
        self.out, self.planes = out, planes

    @property
    def shape(self):
        return self.out.shape


_FUSE_FINALIZE = os.environ.get("CLB200_FUSE_FINALIZE", "1") != "0"


def linear_planes(x, w):
    """``x @ w.T`` for a consumer that accepts ``SplitKPlanes`` (inference only, no autograd): when the GEMM slices
    K, the separate kernel that adds the slices is skipped and the consumer reads the planes."""
    x2 = x.reshape(-1, x.shape[-1])
    if _FUSE_FINALIZE and _GEMM_IMPL == "tcgen05" and not torch.is_grad_enabled() and x2.shape[0] > 0 and _gemm_ok(x2, w) \
            and x.dim() == 2:
        _count("gemm_bf16_nt")
        out, planes = C.gemm_bf16_nt_planes(x2, w)
        return SplitKPlanes(out, planes) if planes.numel() > 0 else out
    return linear(x, w)


@torch.no_grad()
def add_rmsnorm_(resid, delta, w, eps):
    """Residual add + RMSNorm in one pass (inference): ``resid += delta`` in place, returns the norm."""
    if isinstance(delta, SplitKPlanes):
        _count("planes_residual_rmsnorm")
        return C.planes_residual_rmsnorm(resid, delta.planes, w, float(eps))
    H = resid.shape[-1]
    if (resid.dtype != torch.bfloat16 or delta.dtype != torch.bfloat16 or resid.dim() != 2 or H % 8 or H > 8192
            or not resid.is_contiguous() or (w is not None and w.dtype != torch.bfloat16)):
        library_counts["add_rmsnorm_"] += 1
        return ref.add_rmsnorm_(resid, delta, w, eps)
    _count("add_residual_rmsnorm")
    return C.add_residual_rmsnorm(resid, delta.contiguous(), w, float(eps))


# ------------------------------------------------------------------ swiglu
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        guc = gu.contiguous()
        ctx.save_for_backward(guc)
        _count("swiglu_fwd")
        return C.swiglu_fwd(guc)

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        _count("swiglu_bwd")
        return C.swiglu_bwd(gu, dy.contiguous())


def swiglu(gate_up):
    F = gate_up.shape[-1] // 2
    if gate_up.dtype not in (torch.float32, torch.bfloat16) or F % (16 // gate_up.element_size()) != 0:
        library_counts["swiglu"] += 1
        return ref.swiglu(gate_up)
    return _SwiGLU.apply(gate_up)


# ------------------------------------------------------------------ qk-norm + rope
_inv_freq_cache = {}


def _inv_freq(d, theta, device):
    key = (d, float(theta), str(device))
    t = _inv_freq_cache.get(key)
    if t is None:
        t = 1.0 / (theta ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
        _inv_freq_cache[key] = t
    return t


class _NormRope(torch.autograd.Function):
    """Per-head RMSNorm (optional) + rotate-half RoPE on ``x [T, n, D]`` (any row stride)."""

    @staticmethod
    def forward(ctx, x, w, positions, theta, eps):
        T, n, D = x.shape
        x2 = x.reshape(T, n * D) if x.is_contiguous() else x.as_strided((T, n * D), (x.stride(0), 1))
        inv = _inv_freq(D, theta, x.device)
        pos = positions.to(torch.int64)
        out = C.qk_norm_rope_fwd(x2, n, D, w, pos, inv, eps)
        _count("qk_norm_rope_fwd")
        ctx.save_for_backward(x2, w if w is not None else torch.empty(0, device=x.device), pos, inv)
        ctx.has_w, ctx.n, ctx.D, ctx.eps = w is not None, n, D, eps
        return out

    @staticmethod
    def backward(ctx, dy):
        x2, w, pos, inv = ctx.saved_tensors
        T = x2.shape[0]
        dx = torch.empty(T, ctx.n * ctx.D, dtype=x2.dtype, device=x2.device)
        dw = C.qk_norm_rope_bwd(dy.contiguous(), x2, dx, ctx.n, ctx.D, w if ctx.has_w else None, pos, inv, ctx.eps)
        _count("qk_norm_rope_bwd")
        return dx.view(T, ctx.n, ctx.D), (dw.to(w.dtype) if ctx.has_w else None), None, None, None


def _rope_ok(x):
    return (x.dim() == 3 and x.shape[-1] in (64, 128) and x.stride(-1) == 1 and x.stride(1) == x.shape[-1]
            and x.dtype in (torch.float32, torch.bfloat16))


def qk_norm_rope(q, k, qw, kw, eps, positions, theta):
    if not (_rope_ok(q) and _rope_ok(k)):
        library_counts["qk_norm_rope"] += 1
        return ref.qk_norm_rope(q, k, qw, kw, eps, positions, theta)
    return (_NormRope.apply(q, qw, positions, theta, eps), _NormRope.apply(k, kw, positions, theta, eps))


@torch.no_grad()
def qkv_rope_append(qkv, nq, nkv, D, q_weight, k_weight, eps, positions, theta, slot_mapping, k_cache, v_cache):
    """One kernel for q/k norm + RoPE and the cache append (see ``reference.qkv_rope_append``)."""
    planes = None
    if isinstance(qkv, SplitKPlanes):
        qkv, planes = qkv.out, qkv.planes
    ok = (qkv.dtype == torch.bfloat16 and qkv.dim() == 2 and qkv.stride(1) == 1 and D in (64, 128)
          and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16 and k_cache.is_contiguous()
          and v_cache.is_contiguous() and k_cache.shape[-1] == D and v_cache.shape[-1] == D
          and (q_weight is None) == (k_weight is None)
          and (q_weight is None or (q_weight.dtype == torch.bfloat16 and k_weight.dtype == torch.bfloat16)))
    if not ok:
        library_counts["qkv_rope_append"] += 1
        return ref.qkv_rope_append(qkv, nq, nkv, D, q_weight, k_weight, eps, positions, theta, slot_mapping, k_cache,
                                   v_cache)
    _count("qkv_rope_append")
    return C.qkv_rope_append(qkv, nq, nkv, D, q_weight, k_weight, positions.to(torch.int64),
                             _inv_freq(D, theta, qkv.device), slot_mapping.to(torch.int64), k_cache, v_cache, float(eps),
                             planes)


def rope(x, positions, theta, rot_dim=None):
    if (rot_dim is not None and rot_dim != x.shape[-1]) or not _rope_ok(x):
        library_counts["rope"] += 1
        return ref.rope(x, positions, theta, rot_dim)
    return _NormRope.apply(x, None, positions, theta, 0.0)


# ------------------------------------------------------------------ linear / GEMM
def _row_major_ok(t):
    return t.stride(-1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def _main_grad(w):
    """The fp32 accumulation buffer of a parameter (a view of its block's flat gradient buffer), if it has one."""
    g = getattr(w, "main_grad", None)
    if g is not None and g.dtype == torch.float32 and g.is_contiguous() and g.shape == w.shape and g.data_ptr() % 16 == 0:
        return g
    return None


def wgrad_accumulate(dy, x, w):
    """Weight gradient ``dy^T x`` of ``y = x w^T`` on the tcgen05 kernel.  Where the parameter has an fp32
    accumulation buffer the kernel adds into it in its epilogue (no bf16 gradient, no separate add) and
    ``None`` is returned for autograd; otherwise the bf16 gradient is returned."""
    main = _main_grad(w)
    _count("gemm_bf16_tn")
    if main is not None:
        C.gemm_bf16_tn(dy, x, main, True, True)
        return None
    return C.gemm_bf16_tn(dy, x, None, False, False)


class _LinearNT(torch.autograd.Function):
    """y = x W^T, dx = dy W and dW = dy^T x, all three on the tcgen05 kernel (operand layouts NT, NN, TN)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        _count("gemm_bf16_nt")
        return C.gemm_bf16_nt(x, w, False)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        if not _row_major_ok(dy):
            dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            _count("gemm_bf16_nn")
            dx = C.gemm_bf16_nn(dy, w, False)
        if ctx.needs_input_grad[1]:
            dw = wgrad_accumulate(dy, x, w)
        return dx, dw


def _gemm_ok(x2, w):
    return (x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2
            and x2.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0 and x2.stride(-1) == 1 and w.stride(-1) == 1
            and x2.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x2.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def linear(x, w, bias=None):
    if _GEMM_IMPL == "tcgen05":
        x2 = x.reshape(-1, x.shape[-1])
        if x2.shape[0] > 0 and _gemm_ok(x2, w):
            y = _LinearNT.apply(x2, w).view(*x.shape[:-1], w.shape[0])
            return y + bias if bias is not None else y
    library_counts["linear"] += 1
    return torch.nn.functional.linear(x, w, bias)


def linear_out(x2, w, out):
    """``out[:] = x2 @ w.T`` into a caller-owned buffer (no autograd)."""
    if _GEMM_IMPL == "tcgen05" and x2.shape[0] > 0 and _gemm_ok(x2, w):
        _count("gemm_bf16_nt")
        C.gemm_bf16_nt_out(x2, w, out)
    else:
        library_counts["linear"] += 1
        torch.mm(x2, w.t(), out=out)
    return out


def push_ok(x2, w):
    return _GEMM_IMPL == "tcgen05" and x2.shape[0] > 0 and _gemm_ok(x2, w)


def linear_push(x2, w, out, dst_ptrs):
    """``x2 @ w.T`` stored by the GEMM epilogue to every address of ``dst_ptrs`` (the copies of a
    symmetric staging slot on all ranks of a group, peers' memory included); ``out`` is this
    rank's copy."""
    _count("gemm_bf16_nt_push")
    C.gemm_bf16_nt_push(x2, w, out, [int(p) for p in dst_ptrs])
    return out


def gemm_nt(a, b, out_fp32=False):
    """Raw C = A B^T on the tcgen05 kernel (no autograd)."""
    _count("gemm_bf16_nt")
    return C.gemm_bf16_nt(a, b, out_fp32)


def gemm_nn(a, b, out_fp32=False):
    """Raw C[M, N] = A[M, K] B[K, N] (both row-major) on the tcgen05 kernel (no autograd)."""
    _count("gemm_bf16_nn")
    return C.gemm_bf16_nn(a, b, out_fp32)


def gemm_tn(a, b, out=None, accumulate=False, out_fp32=False):
    """Raw C[M, N] (+)= A[K, M]^T B[K, N] (both row-major) on the tcgen05 kernel (no autograd)."""
    _count("gemm_bf16_tn")
    return C.gemm_bf16_tn(a, b, out, accumulate, out_fp32)


# ------------------------------------------------------------------ lm head log-prob / entropy
class _LMHeadLogprob(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels, inv_temp, chunk):
        T = h.shape[0]
        lp = torch.empty(T, dtype=torch.float32, device=h.device)
        ent = torch.empty(T, dtype=torch.float32, device=h.device)
        lse = torch.empty(T, dtype=torch.float32, device=h.device)
        lab = labels.to(torch.int64).contiguous()
        use_own = _GEMM_IMPL == "tcgen05" and _gemm_ok(h, w)
        for s in range(0, T, chunk):
            hc = h[s:s + chunk]
            if use_own:
                z = C.gemm_bf16_nt(hc, w, True)
                _count("gemm_bf16_nt")
            else:
                z = (hc @ w.t()).float() if hc.dtype != torch.float32 else hc @ w.t()
            a, b, c = C.logits_stats(z.contiguous(), lab[s:s + chunk], inv_temp)
            _count("logits_stats")
            lp[s:s + chunk], ent[s:s + chunk], lse[s:s + chunk] = a, b, c
        ctx.save_for_backward(h, w, lab, lse, ent)
        ctx.inv_temp, ctx.chunk, ctx.use_own = inv_temp, chunk, use_own
        ctx.mark_non_differentiable(lse)
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        h, w, lab, lse, ent = ctx.saved_tensors
        T = h.shape[0]
        chunk = ctx.chunk
        gh = torch.empty_like(h)
        own_bwd = ctx.use_own and h.dtype == torch.bfloat16
        # the weight gradient is accumulated by the GEMM epilogue: straight into the parameter's fp32
        # accumulation buffer where it has one, else into a local fp32 buffer
        main = _main_grad(w) if own_bwd else None
        gw = main if main is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        g_lp = g_lp.contiguous().float()
        ge = g_ent.contiguous().float() if g_ent is not None else None
        bf = h.dtype == torch.bfloat16
        for s in range(0, T, chunk):
            hc = h[s:s + chunk]
            if ctx.use_own:
                z = C.gemm_bf16_nt(hc, w, True)
                _count("gemm_bf16_nt")
            else:
                z = (hc @ w.t()).float() if hc.dtype != torch.float32 else hc @ w.t()
            dz = C.logits_grad(z.contiguous(), lab[s:s + chunk], lse[s:s + chunk], ent[s:s + chunk],
                               g_lp[s:s + chunk], ge[s:s + chunk] if ge is not None else None,
                               ctx.inv_temp, bf)
            _count("logits_grad")
            if own_bwd:
                gh[s:s + chunk] = C.gemm_bf16_nn(dz, w, False)
                C.gemm_bf16_tn(dz, hc, gw, True, True)
                _count("gemm_bf16_nn")
                _count("gemm_bf16_tn")
            else:
                library_counts["lmhead_backward_mm"] += 2
                gh[s:s + chunk] = dz @ w
                gw += (dz.t() @ hc).float()
        return gh, (None if main is not None else gw.to(w.dtype)), None, None, None


def lmhead_logprob_entropy(h, w, labels, temperature=1.0, chunk=2048):
    return _LMHeadLogprob.apply(h.contiguous(), w, labels, 1.0 / temperature, chunk)


# ------------------------------------------------------------------ GRPO loss
class _GrpoLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lp, old, ref_lp, adv, mask, ent, pos_clip, neg_clip, diff_clip, final_clip, kl_coef,
                ent_coef, inv_norm):
        f = lambda t: None if t is None else t.contiguous().float()  # noqa: E731
        stats, dlp, dent = C.grpo_loss_fwd(f(lp), f(old), f(ref_lp), f(adv), f(mask), f(ent), pos_clip,
                                           neg_clip, diff_clip, final_clip, kl_coef, ent_coef, inv_norm)
        _count("grpo_loss")
        ctx.save_for_backward(dlp, dent)
        ctx.has_ent = ent is not None
        total = stats[6] * inv_norm
        ctx.mark_non_differentiable(stats)
        return total, stats[:6]

    @staticmethod
    def backward(ctx, g_total, _g_stats):
        dlp, dent = ctx.saved_tensors
        g_ent = dent * g_total if ctx.has_ent and dent.numel() else None
        return (dlp * g_total, None, None, None, None, g_ent) + (None,) * 7


def grpo_loss_fused(logprobs, old_logprobs, ref_logprobs, advantages, mask, entropy=None, pos_clip=0.2,
                    neg_clip=0.2, diff_clip=10.0, final_clip=3.0, kl_coef=0.0, entropy_coef=0.0, inv_norm=1.0):
    adv = advantages if advantages.shape == logprobs.shape else advantages.expand_as(logprobs)
    return _GrpoLoss.apply(logprobs, old_logprobs, ref_logprobs, adv, mask, entropy, pos_clip, neg_clip,
                           diff_clip, final_clip, kl_coef, entropy_coef, inv_norm)


class _GspoLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lp, old, ref_lp, adv, mask, ent, seq_ids, num_seqs, pos_clip, neg_clip, diff_clip, final_clip,
                kl_coef, ent_coef, inv_norm):
        f = lambda t: None if t is None else t.contiguous().float()  # noqa: E731
        stats, dlp, dent = C.gspo_loss_fwd(f(lp), f(old), f(ref_lp), f(adv), f(mask), f(ent),
                                           seq_ids.to(torch.int64).contiguous(), int(num_seqs), pos_clip, neg_clip,
                                           diff_clip, final_clip, kl_coef, ent_coef, inv_norm)
        _count("gspo_loss", 2)
        ctx.save_for_backward(dlp, dent)
        ctx.has_ent = ent is not None
        total = stats[6] * inv_norm
        ctx.mark_non_differentiable(stats)
        return total, stats[:6]

    @staticmethod
    def backward(ctx, g_total, _g_stats):
        dlp, dent = ctx.saved_tensors
        g_ent = dent * g_total if ctx.has_ent and dent.numel() else None
        return (dlp * g_total, None, None, None, None, g_ent) + (None,) * 9


def gspo_loss_fused(logprobs, old_logprobs, ref_logprobs, advantages, mask, seq_ids, num_seqs, entropy=None,
                    pos_clip=3e-4, neg_clip=4e-4, diff_clip=10.0, final_clip=3.0, kl_coef=0.0, entropy_coef=0.0,
                    inv_norm=1.0):
    adv = advantages if advantages.shape == logprobs.shape else advantages.expand_as(logprobs)
    return _GspoLoss.apply(logprobs, old_logprobs, ref_logprobs, adv, mask, entropy, seq_ids, num_seqs, pos_clip,
                           neg_clip, diff_clip, final_clip, kl_coef, entropy_coef, inv_norm)


# ------------------------------------------------------------------ optimizer
@torch.no_grad()
def adamw_step(master, grad, exp_avg, exp_avg_sq, out_param, step, lr, beta1, beta2, eps, weight_decay,
               grad_scale=1.0):
    ok = (master.dtype == torch.float32 and grad.dtype == torch.float32 and master.is_contiguous()
          and grad.is_contiguous() and all(t.data_ptr() % 16 == 0 for t in (master, grad, exp_avg, exp_avg_sq))
          and (out_param is None or (out_param.is_contiguous() and out_param.dtype in (torch.float32, torch.bfloat16))))
    if not ok:
        library_counts["adamw_step"] += 1
        return ref.adamw_step(master, grad, exp_avg, exp_avg_sq, out_param, step, lr, beta1, beta2, eps,
                              weight_decay, grad_scale)
    if isinstance(grad_scale, torch.Tensor):
        st, sv = grad_scale.reshape(1).float(), 1.0
    else:
        st, sv = None, float(grad_scale)
    C.adamw_step(master, grad, exp_avg, exp_avg_sq, out_param, int(step), lr, beta1, beta2, eps, weight_decay,
                 st, sv)
    _count("adamw_step")


@torch.no_grad()
def sumsq(x):
    if x.dtype not in (torch.float32, torch.bfloat16):
        return ref.sumsq(x)
    _count("sumsq", 2)
    return C.sumsq(x)


# ------------------------------------------------------------------ sampling
@torch.no_grad()
def sample(logits, u, temperature=1.0, top_k=-1, top_p=1.0, min_p=0.0):
    z = logits.float().contiguous()
    ids, lp = C.sample(z, u.float().contiguous(), float(temperature), int(top_k if top_k is not None else -1),
                       float(top_p), float(min_p))
    _count("sample")
    return ids, lp


@torch.no_grad()
def apply_penalties(logits, token_counts, presence=0.0, frequency=0.0, repetition=1.0, prompt_mask=None):
    _count("apply_penalties")
    return C.apply_penalties(logits, token_counts, prompt_mask, presence, frequency, repetition)


# ------------------------------------------------------------------ paged KV cache
@torch.no_grad()
def kv_append(k, v, k_cache, v_cache, slot_mapping):
    if k.dtype != k_cache.dtype or k.dtype not in (torch.float32, torch.bfloat16):
        library_counts["kv_append"] += 1
        return ref.kv_append(k, v, k_cache, v_cache, slot_mapping)
    kk = k if (k.stride(2) == 1 and k.stride(1) == k.shape[2]) else k.contiguous()
    vv = v if (v.stride(2) == 1 and v.stride(1) == v.shape[2]) else v.contiguous()
    C.kv_append(kk, vv, k_cache, v_cache, slot_mapping.to(torch.int64))
    _count("kv_append")


_DECODE_IMPL = os.environ.get("CHATLEARN_DECODE", "tc")   # "tc" | "simt"


def set_decode_impl(name: str):
    global _DECODE_IMPL
    assert name in ("tc", "simt")
    _DECODE_IMPL = name


def _num_splits(n_ctas: int, max_ctx_blocks: int) -> int:
    """Split long contexts when the grid alone cannot fill the 148 SMs."""
    if n_ctas >= 148 * 2 or max_ctx_blocks <= 4:
        return 1
    return int(max(1, min(max_ctx_blocks // 2, (148 * 2 + n_ctas - 1) // n_ctas, 16)))


@torch.no_grad()
def paged_attention(q, k_cache, v_cache, block_tables, seq_lens, q_lens=None, scale=None, groups=None):
    nb, bs, nkv, dk = k_cache.shape
    dv = v_cache.shape[-1]
    nq = q.shape[1]
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or \
            not C.paged_decode_supported(dk, dv, bs, nq // nkv):
        library_counts["paged_attention"] += 1
        if (q_lens is None or q.shape[0] == seq_lens.shape[0]) and q.shape[0] > 0:
            # decode rows: batched statements without host synchronisation, so the step can still be captured
            from .paged_fallback import paged_decode_batched
            return paged_decode_batched(q, k_cache, v_cache, block_tables, seq_lens,
                                        scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]))
        return ref.paged_attention(q, k_cache, v_cache, block_tables, seq_lens, q_lens, scale)
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    sl = seq_lens.to(torch.int32)
    if (groups is not None and (q_lens is None or q.shape[0] == sl.shape[0]) and _DECODE_IMPL == "tc"
            and dk == 128 and dv == 128 and bs == 64 and nq // nkv <= 4):
        # sequences that adopted the same prompt blocks: the shared blocks are attended once per group (all members'
        # queries as rows of one MMA tile), the rest per sequence, merged by log-sum-exp
        grp_q, grp_nblk, blk_start = groups
        _count("paged_decode_grouped", 3)
        return C.paged_decode_tc_grouped(q.contiguous(), k_cache, v_cache, block_tables.to(torch.int32).contiguous(), sl,
                                         grp_q, grp_nblk, blk_start, float(scale), 2, 1)
    if q_lens is None or q.shape[0] == sl.shape[0]:
        q_seq, ctx = None, sl
    else:
        ql = q_lens.to(torch.int64)
        B = sl.shape[0]
        q_seq = torch.repeat_interleave(torch.arange(B, device=q.device, dtype=torch.int32), ql)
        ends = torch.cumsum(ql, 0)
        idx = torch.arange(q.shape[0], device=q.device)
        back = (ends[q_seq.long()] - 1 - idx).to(torch.int32)      # tokens after this one in its chunk
        ctx = sl[q_seq.long()] - back
    max_blocks = block_tables.shape[1]
    ns = _num_splits(q.shape[0] * nkv, max_blocks)
    _count("paged_decode", 1 if ns == 1 else 2)
    # tensor-core kernel for 64-token blocks; the SIMT kernel covers the other block sizes
    fn = C.paged_decode_tc if (_DECODE_IMPL == "tc" and C.paged_decode_tc_supported(dk, dv, bs, nq // nkv)) \
        else C.paged_decode
    return fn(q.contiguous(), k_cache, v_cache, block_tables.to(torch.int32).contiguous(), q_seq,
              ctx.contiguous(), float(scale), ns)


def mla_paged_decode(q, k_cache, lora, block_tables, seq_lens, scale):
    """Latent-attention decode on the tensor-core kernel (latent 512 + rotary 64, 64-row blocks, bf16); other
    shapes run the batched statements."""
    D = q.shape[-1]
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or lora != 512 or D != 576 or k_cache.shape[1] != 64:
        library_counts["mla_paged_decode"] += 1
        return ref.mla_paged_decode(q, k_cache, lora, block_tables, seq_lens, scale)
    _count("mla_decode")
    return C.mla_paged_decode(q.contiguous(), k_cache, block_tables.to(torch.int32).contiguous(),
                              seq_lens.to(torch.int32).contiguous(), float(scale), 0)


# ------------------------------------------------------------------ weight sync kernel
def weight_sync_run(desc_table, num_descs, total_tiles, src_dtype, dst_dtype):
    C.weight_sync_run(desc_table, num_descs, total_tiles, src_dtype, dst_dtype)
    _count("weight_sync")


for _name, _fn in (("rmsnorm", rmsnorm), ("add_rmsnorm_", add_rmsnorm_), ("swiglu", swiglu), ("qk_norm_rope", qk_norm_rope), ("qkv_rope_append", qkv_rope_append), ("rope", rope),
                   ("linear", linear), ("lmhead_logprob_entropy", lmhead_logprob_entropy),
                   ("grpo_loss_fused", grpo_loss_fused), ("gspo_loss_fused", gspo_loss_fused), ("adamw_step", adamw_step), ("sumsq", sumsq),
                   ("sample", sample), ("apply_penalties", apply_penalties), ("kv_append", kv_append),
                   ("paged_attention", paged_attention), ("mla_paged_decode", mla_paged_decode),
                   ("linear_planes", linear_planes)):
    register_native(_name, _fn)

from . import native_moe  # noqa: E402,F401  (registers the mixture-of-experts ops)
from . import native_attn  # noqa: E402,F401  (registers the packed attention forward)
