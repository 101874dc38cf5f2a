"""Mixture-of-experts ops on the sm_100a kernels.

router            csrc/moe.cu  moe_router_topk (scores, group-limited top-k, weights, histogram)
dispatch          csrc/moe.cu  moe_permute (rows sorted by expert, no host round trip)
expert MLPs       csrc/gemm_sm100.cu  grouped tcgen05 GEMM driven by a device-built tile table
combine           csrc/moe.cu  moe_combine (fp32 weighted sum of the k expert outputs)

The reference gets these from TransformerEngine (grouped GEMM, permute/unpermute:
chatlearn/models/patches/transformers/layers/groupgemm.py:65-208) and from eager torch
(router: qwen3_moe_patch.py:36-43).  Backward passes run here as well: routing
gradients are closed-form; the expert GEMMs' input and weight gradients run on the same
grouped kernel (every expert's rows padded to a multiple of 64 in the sorted layout, so
the weight gradient's contraction over an expert's rows never touches a neighbour's).
Rows that arrive densely packed from the expert-parallel exchange (``grouped_mlp``) keep
the per-expert library GEMMs after one read-back of the group sizes.
"""
import os

import torch

from . import library_counts, reference as ref, register_native
from . import native as _n

C = _n.C
_count = _n._count


# ------------------------------------------------------------------ router
class _Router(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, k, sigmoid, norm, n_group, topk_group, scale):
        w, idx, scores, hist = C.moe_router_topk(logits.contiguous(), k, sigmoid, norm, bias, n_group, topk_group, scale)
        _count("moe_router_topk")
        ctx.save_for_backward(scores, idx)
        ctx.cfg = (sigmoid, norm, scale, logits.dtype)
        ctx.mark_non_differentiable(idx, hist)
        return w, idx, scores, hist

    @staticmethod
    def backward(ctx, gw, _gi, gs, _gh):
        scores, idx = ctx.saved_tensors
        sigmoid, norm, scale, dtype = ctx.cfg
        ds = gs.float().clone() if gs is not None else torch.zeros_like(scores)
        if gw is not None:
            gw = gw.float()
            raw = scores.gather(1, idx)
            if norm:
                S = raw.sum(-1, keepdim=True) + 1e-20
                draw = scale * (gw / S - (gw * raw).sum(-1, keepdim=True) / (S * S))
            else:
                draw = scale * gw
            ds.scatter_add_(1, idx, draw)
        if sigmoid:
            dz = ds * scores * (1 - scores)
        else:
            dz = scores * (ds - (ds * scores).sum(-1, keepdim=True))
        return dz.to(dtype), None, None, None, None, None, None, None


def moe_router(logits, top_k, scoring="softmax", norm_topk=True, bias=None, n_group=1, topk_group=1, scale=1.0):
    E = logits.shape[-1]
    if logits.dim() != 2 or E > 512 or top_k > 16 or n_group > 16 or logits.dtype not in (torch.float32, torch.bfloat16):
        library_counts["moe_router"] += 1
        return ref.moe_router(logits, top_k, scoring, norm_topk, bias, n_group, topk_group, scale)
    w, idx, scores, hist = _Router.apply(logits, bias, int(top_k), scoring != "softmax", bool(norm_topk),
                                         int(n_group), int(topk_group), float(scale))
    idx._moe_hist = hist              # tokens per expert, reused by the dispatch
    return w, idx, scores


# ------------------------------------------------------------------ dispatch / combine
_PAD = 64     # every expert's rows start at a multiple of the K tile of the weight-gradient GEMM
# "grouped": backward on the grouped tcgen05 kernels; "library": per-expert library GEMMs (kept for comparison)
_BWD_IMPL = os.environ.get("CLB200_MOE_BWD", "grouped")


def _offsets(idx, num_experts, pad: int = 1):
    """First row of every expert in the sorted layout (device tensor, no host read-back).  ``pad`` > 1 rounds every
    expert's row count up to a multiple of it; the rows in between stay zero."""
    hist = getattr(idx, "_moe_hist", None)
    if hist is None or hist.numel() != num_experts:
        hist = torch.bincount(idx.reshape(-1), minlength=num_experts)
    if pad > 1:
        hist = (hist + (pad - 1)) // pad * pad
    off = torch.zeros(num_experts + 1, dtype=torch.long, device=idx.device)
    off[1:] = hist.cumsum(0)
    return off


class _Permute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx, offsets, total_rows=-1):
        xs, pos = C.moe_permute(x.contiguous(), idx.contiguous(), offsets, int(total_rows))
        _count("moe_permute")
        ctx.save_for_backward(pos)
        ctx.mark_non_differentiable(pos)
        return xs, pos

    @staticmethod
    def backward(ctx, dxs, _):
        (pos,) = ctx.saved_tensors
        _count("moe_combine")
        return C.moe_combine(dxs.contiguous(), pos, None), None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ys, pos, weights):
        ctx.save_for_backward(ys, pos, weights)
        _count("moe_combine")
        return C.moe_combine(ys.contiguous(), pos, weights)

    @staticmethod
    def backward(ctx, dy):
        ys, pos, weights = ctx.saved_tensors
        dy = dy.contiguous()
        _count("moe_permute")
        # same row layout as ys (padded or not); rows no pair maps to are zero
        dys = C.moe_permute_at(dy, pos, weights, int(ys.shape[0]) if ys.shape[0] != pos.numel() else -1)
        _count("moe_row_dot")
        dw = C.moe_row_dot(dy, ys, pos)
        return dys, None, dw.to(weights.dtype)


class _GroupedMLP(torch.autograd.Function):
    """SwiGLU expert MLPs over rows sorted by expert (``offsets`` on the device).

    ``padded``: every expert's rows start at a multiple of 64 and the rows between two experts are zero.  The
    backward then runs on the grouped tcgen05 GEMMs as well (input gradients: the forward's tile table with the
    weights read in their stored layout; weight gradients: one tile per (expert, 128 x 256 block of its weight),
    contraction over the expert's rows), with no read-back of the group sizes.  Otherwise (rows packed densely,
    as the expert-parallel exchange delivers them) the backward loops over the experts on library GEMMs."""

    @staticmethod
    def forward(ctx, xs, w13, w2, offsets, padded=False):
        h13 = C.grouped_gemm_bf16_nt(xs, w13, offsets)
        act = C.swiglu_fwd(h13)
        ys = C.grouped_gemm_bf16_nt(act, w2, offsets)
        _count("grouped_gemm_bf16_nt", 2)
        _count("swiglu_fwd")
        ctx.save_for_backward(xs, w13, w2, offsets, h13)
        ctx.padded = bool(padded) and w13.shape[1] % 64 == 0 and w2.shape[1] % 64 == 0
        return ys

    @staticmethod
    def backward(ctx, dys):
        xs, w13, w2, offsets, h13 = ctx.saved_tensors
        dys = dys.contiguous()
        if ctx.padded:
            act = C.swiglu_fwd(h13)
            dact = C.grouped_gemm_bf16_nn(dys, w2, offsets)                               # [R, F]
            dw2 = C.grouped_gemm_bf16_tn(dys, act, offsets, torch.empty_like(w2), False)  # [E, H, F]
            dh13 = C.swiglu_bwd(h13, dact)
            dxs = C.grouped_gemm_bf16_nn(dh13, w13, offsets)                              # [R, H]
            dw13 = C.grouped_gemm_bf16_tn(dh13, xs, offsets, torch.empty_like(w13), False)
            _count("grouped_gemm_bf16_nn", 2)
            _count("grouped_gemm_bf16_tn", 2)
            _count("swiglu_fwd")
            _count("swiglu_bwd")
            return dxs, dw13, dw2, None, None
        bounds = offsets.tolist()                      # one read-back per layer
        act = C.swiglu_fwd(h13)
        dact = torch.empty_like(act)
        dw2 = torch.zeros_like(w2)
        for e in range(w2.shape[0]):
            s, t = bounds[e], bounds[e + 1]
            if t > s:
                torch.mm(dys[s:t], w2[e], out=dact[s:t])
                torch.mm(dys[s:t].t(), act[s:t], out=dw2[e])
        dh13 = C.swiglu_bwd(h13, dact)
        dxs = torch.zeros_like(xs)
        dw13 = torch.zeros_like(w13)
        for e in range(w13.shape[0]):
            s, t = bounds[e], bounds[e + 1]
            if t > s:
                torch.mm(dh13[s:t], w13[e], out=dxs[s:t])
                torch.mm(dh13[s:t].t(), xs[s:t], out=dw13[e])
        library_counts["grouped_gemm_bwd"] += 1
        return dxs, dw13, dw2, None, None


def _moe_ok(x, w13, w2):
    return (x.dtype == torch.bfloat16 and w13.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16 and x.dim() == 2
            and x.shape[1] % 8 == 0 and w13.shape[1] % 16 == 0 and w2.shape[2] % 8 == 0 and w13.shape[0] <= 1024
            and w13.is_contiguous() and w2.is_contiguous())


def grouped_mlp(xs, w13, w2, counts):
    if not _moe_ok(xs, w13, w2) or xs.shape[0] == 0:
        library_counts["grouped_mlp"] += 1
        return ref.grouped_mlp(xs, w13, w2, counts)
    c = torch.tensor(counts, dtype=torch.long)
    off = torch.zeros(len(counts) + 1, dtype=torch.long)
    off[1:] = c.cumsum(0)
    if torch.is_grad_enabled() and (xs.requires_grad or w13.requires_grad) and _BWD_IMPL == "grouped" \
            and w13.shape[1] % 64 == 0 and w2.shape[1] % 64 == 0:
        # training: move the rows into the layout whose groups start at multiples of 64 (zero rows in between),
        # so that the backward runs on the grouped kernels; the group sizes are on the host already
        p = (c + (_PAD - 1)) // _PAD * _PAD
        poff = torch.zeros(len(counts) + 1, dtype=torch.long)
        poff[1:] = p.cumsum(0)
        R, dev = xs.shape[0], xs.device
        shift = (poff[:-1] - off[:-1]).to(dev, non_blocking=True)
        keep = torch.arange(R, device=dev) + torch.repeat_interleave(shift, c.to(dev, non_blocking=True), output_size=R)
        xs_pad = xs.new_zeros(int(poff[-1]), xs.shape[1]).index_copy(0, keep, xs)
        ys = _GroupedMLP.apply(xs_pad, w13, w2, poff.to(dev, non_blocking=True), True)
        return ys.index_select(0, keep)
    return _GroupedMLP.apply(xs.contiguous(), w13, w2, off.to(xs.device, non_blocking=True))


def moe_experts(x, w13, w2, weights, idx):
    if not _moe_ok(x, w13, w2) or x.shape[0] == 0:
        library_counts["moe_experts"] += 1
        return ref.moe_experts(x, w13, w2, weights, idx)
    E = w13.shape[0]
    if torch.is_grad_enabled() and (x.requires_grad or w13.requires_grad) and _BWD_IMPL == "grouped":
        # training: padded groups, so that the backward runs on the grouped kernels too
        offsets = _offsets(idx, E, _PAD)
        xs, pos = _Permute.apply(x, idx, offsets, idx.numel() + E * _PAD)
        ys = _GroupedMLP.apply(xs, w13, w2, offsets, True)
    else:
        offsets = _offsets(idx, E)
        xs, pos = _Permute.apply(x, idx, offsets)
        ys = _GroupedMLP.apply(xs, w13, w2, offsets)
    return _Combine.apply(ys, pos, weights.float())


for _name, _fn in (("moe_router", moe_router), ("moe_experts", moe_experts), ("grouped_mlp", grouped_mlp)):
    register_native(_name, _fn)
