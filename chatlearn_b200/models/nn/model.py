"""Decoder-only transformer written as functions over flat parameter blocks.

One implementation serves the trainer (packed varlen batches, autograd), the
reference/reward roles (no-grad forward) and the rollout engine (paged KV
cache), for Llama-2, Qwen2/Qwen3 dense, Qwen3-MoE and DeepSeek-V3/Moonlight
(MLA + shared-expert MoE).  Parameters live in one contiguous buffer per block
(embedding, each decoder layer, head); the block is the unit of sharding,
all-gather/reduce-scatter, offload and weight sync.  The reference relies on
HF ``AutoModelForCausalLM`` (chatlearn/models/fsdp_module.py:250-295) or
Megatron-Core ``GPTModel``; neither is used here.
"""
import math
import zlib
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from chatlearn_b200 import ops
from .arch import ModelArch
from .layout import Leaf, model_blocks

ALIGN = 128  # leaf offsets inside a block are multiples of this many elements (TMA/vector alignment)


def _align(n, a=ALIGN):
    return (n + a - 1) // a * a


class ParamBlock:
    """Leaves of one block laid out in one flat tensor."""

    def __init__(self, name: str, leaves: List[Leaf], dtype, device, pad_to: int = 1,
                 allocate: bool = True):
        self.name, self.leaves = name, leaves
        self.offsets: Dict[str, int] = {}
        off = 0
        for lf in leaves:
            self.offsets[lf.name] = off
            off += _align(lf.numel)
        self.numel = _align(off, ALIGN * pad_to)
        self.dtype, self.device = dtype, device
        self.flat: Optional[torch.Tensor] = None
        self.grad: Optional[torch.Tensor] = None
        self.params: Dict[str, torch.Tensor] = {}
        if allocate:
            self.bind(torch.zeros(self.numel, dtype=dtype, device=device))

    def short(self, leaf_name: str) -> str:
        return leaf_name.split(".", 2)[-1] if leaf_name.startswith("layers.") else leaf_name

    def bind(self, flat: torch.Tensor):
        """Point every leaf at ``flat`` (shape ``[numel]``)."""
        assert flat.numel() == self.numel
        self.flat = flat
        for lf in self.leaves:
            o = self.offsets[lf.name]
            # detach(): the leaf must not keep a `_base` reference to the flat buffer,
            # or re-pointing its `.data` (offload) would not release the memory
            view = flat[o:o + lf.numel].view(lf.shape).detach()
            key = self.short(lf.name)
            if key in self.params:
                self.params[key].data = view
            else:
                self.params[key] = view
        return self

    def enable_grad(self, grad_flat: torch.Tensor):
        """Make leaves autograd leaves whose ``.grad`` are views of ``grad_flat``:
        autograd accumulates into them in place, so the block's gradient is one
        contiguous buffer ready for reduce-scatter."""
        for lf in self.leaves:
            key = self.short(lf.name)
            p = self.params[key]
            if not p.requires_grad:
                p = p.detach().requires_grad_(True)
                self.params[key] = p
            o = self.offsets[lf.name]
            gview = grad_flat[o:o + lf.numel].view(lf.shape)
            if grad_flat.dtype == p.dtype:
                p.grad = gview
            elif not getattr(p, "_main_grad_hooked", False):
                # wider accumulation buffer than the parameter dtype: fold each
                # micro-batch gradient into it right after autograd produced it
                p.main_grad = gview
                p._main_grad_hooked = True

                def _fold(param):
                    # a GEMM epilogue may already have added this gradient into main_grad
                    # (ops.native.wgrad_accumulate): then autograd hands over nothing
                    if param.grad is not None:
                        param.main_grad.add_(param.grad)
                        param.grad = None
                p.register_post_accumulate_grad_hook(_fold)
            else:
                p.main_grad = gview

    def leaf_view(self, flat: torch.Tensor, lf: Leaf) -> torch.Tensor:
        o = self.offsets[lf.name]
        return flat[o:o + lf.numel].view(lf.shape)

    @torch.no_grad()
    def init_weights(self, seed: int, std: float = 0.02):
        """Deterministic per-leaf initialisation: the generator of each leaf is
        seeded from (seed, HF tensor names), values are drawn for the *full* HF
        tensor on CPU only for small tensors; large leaves draw on their device."""
        for lf in self.leaves:
            p = self.leaf_view(self.flat, lf)
            if lf.init == "ones":
                p.fill_(1.0)
            elif lf.init == "zeros":
                p.zero_()
            elif lf.init in ("a_log", "conv"):
                # gated delta-net: decay rates A ~ U(1, 16) stored as log A; depthwise conv taps ~ U(-1/sqrt(k), 1/sqrt(k))
                g = torch.Generator(device="cpu")
                g.manual_seed((seed * 1000003 + zlib.crc32(lf.name.encode())) % (2 ** 31))
                u = torch.rand(p.shape, generator=g)
                v = (1.0 + 15.0 * u).log() if lf.init == "a_log" else (2.0 * u - 1.0) / math.sqrt(p.shape[-1])
                p.copy_(v.to(p.device))
            else:
                g = torch.Generator(device=p.device)
                g.manual_seed((seed * 1000003 + zlib.crc32(lf.name.encode())) % (2 ** 31))
                if p.dtype in (torch.float32, torch.bfloat16, torch.float16):
                    p.normal_(0.0, std, generator=g)
                else:
                    p.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device)
                            .normal_(0.0, std, generator=g))


@dataclass
class KVCtx:
    """Paged KV-cache view for one forward of the rollout engine."""
    k_cache: List[torch.Tensor]            # per layer [num_blocks, block, nkv_local, dk]
    v_cache: List[torch.Tensor]
    slot_mapping: torch.Tensor             # [T] flat slot of every new token
    block_tables: torch.Tensor             # [B, max_blocks] int32
    seq_lens: torch.Tensor                 # [B] lengths including the new tokens
    q_lens: Optional[torch.Tensor] = None  # [B] new tokens per sequence (None → 1 each)
    prefill_only: bool = False             # all sequences start at position 0 → varlen kernel
    groups: Any = None                     # decode steps: (group members, shared blocks per group, per-sequence first private block): sequences sharing their prompt blocks
    lin: Any = None                        # models.nn.hybrid.LinearState: conv / recurrent state of gated delta-net layers


@dataclass
class FwdCtx:
    positions: torch.Tensor
    cu_seqlens: Optional[torch.Tensor] = None
    max_seqlen: int = 0
    kv: Optional[KVCtx] = None
    tp: Any = None                         # parallel.groups.Group or None
    ep: Any = None
    sp: Any = None                         # Ulysses sequence-parallel group
    cp: Any = None                         # context-parallel group
    attn_positions: Optional[torch.Tensor] = None  # positions of the rows attention sees (Ulysses)
    cp_plan: Optional[Dict[str, Any]] = None       # ContextParallel.plan() of this packed row
    aux_losses: List[torch.Tensor] = field(default_factory=list)
    aux_weight: Any = None                 # weight of the auxiliary losses in the objective (segment-wise backward passes)
    moe_stats: List[torch.Tensor] = field(default_factory=list)
    tp_symm: Any = None                    # parallel.symm_collectives.SymmGroup of the TP group (inference)
    pending: Any = None                    # sub-layer output (or un-reduced TP partial) not yet added to the residual stream
    fuse_add_norm: bool = False            # inference: fuse residual adds with the following RMSNorm (in-place stream)
    planes_ok: bool = False                # GEMM outputs may be handed on as un-added K-slice planes (set per layer)
    mrope_positions: Optional[torch.Tensor] = None   # [3, T] time/row/column positions (vision-language models)
    deepstack: Any = None                  # (rows, [features per early layer]): vision taps added after layer i (Qwen3-VL)
    seq_parallel: bool = False             # residual stream and norms hold 1/tp of the rows (Megatron sequence parallelism)
    row_valid: Optional[torch.Tensor] = None   # [rows] bool: False for alignment padding (kept out of the balancing loss)


def _tp_reduce(x, ctx):
    """Output of a row-parallel layer: summed over the tensor-parallel group.  Under sequence parallelism
    (Megatron's ``sequence_parallel``: the residual stream and the norms hold 1/tp of the rows) the sum is
    reduce-scattered along the rows instead."""
    if ctx.tp is not None and ctx.tp.size > 1:
        if ctx.seq_parallel:
            return ctx.tp.reduce_scatter_seq(x)
        return ctx.tp.all_reduce(x)
    return x


def _row_parallel(x, w, ctx):
    """Row-parallel linear layer and the sum of its output over the tensor-parallel group.  Under sequence
    parallelism on GPUs the product and the reduce-scatter are one pass (the GEMM epilogue stores every row block
    into its owner's receive buffer over NVLink: ``SymmGroup.gemm_reduce_scatter``)."""
    tp = ctx.tp
    if ctx.planes_ok and (tp is None or tp.size == 1):
        # the caller adds the product to the residual stream in its next kernel, which can read the GEMM's K-slice
        # planes directly
        return ops.linear_planes(x, w)
    if tp is not None and tp.size > 1 and ctx.seq_parallel and x.is_cuda:
        fused = tp.fast.get("gemm_rs")
        if fused is not None:
            y = fused(x, w)
            if y is not None:
                return y
    return _tp_reduce(ops.linear(x, w), ctx)


def attention_block(arch: ModelArch, p: Dict[str, torch.Tensor], x, ctx: FwdCtx, layer: int,
                    partial: bool = False):
    """``partial=True`` (tensor-parallel inference with in-kernel collectives) returns this
    rank's un-reduced output projection, written straight into symmetric staging."""
    d = arch.head_dim
    x = _tp_copy(x, ctx)
    T = x.shape[0]                 # (under sequence parallelism the rows were gathered just now)
    tp = ctx.tp.size if ctx.tp is not None else 1
    nh_l = arch.num_attention_heads // tp
    if arch.use_mla:
        nope, rp, dv = arch.qk_nope_head_dim, arch.qk_rope_head_dim, arch.v_head_dim
        if "q_a_proj" in p:
            qa = ops.rmsnorm(ops.linear(x, p["q_a_proj"]), p["q_a_layernorm"], arch.rms_norm_eps)
            q = ops.linear(qa, p["q_b_proj"])
        else:
            q = ops.linear(x, p["q_proj"])
        q = q.view(T, nh_l, nope + rp)
        ckv = ops.linear(x, p["kv_a_proj_with_mqa"])
        c = ops.rmsnorm(ckv[:, :arch.kv_lora_rank].contiguous(), p["kv_a_layernorm"], arch.rms_norm_eps)
        k_rope = ckv[:, arch.kv_lora_rank:].reshape(T, 1, rp)
        from .mla import attention_scale, rope_decoupled
        q_rope = rope_decoupled(arch, q[..., nope:], ctx.positions)
        k_rope = rope_decoupled(arch, k_rope, ctx.positions)
        q = torch.cat([q[..., :nope], q_rope], dim=-1)
        scale = attention_scale(arch)
        if ctx.kv is not None:
            # rollout: the cache keeps one compressed row per token (normalised latent | rotary key), shared by
            # all heads; steps that read the cache attend in the latent space with the up-projections folded
            # into the query and the output (q·W_uk on the left, ·W_uv on the right of a 1-head attention)
            kvc = ctx.kv
            kc = kvc.k_cache[layer]
            lat = torch.cat([c, k_rope.reshape(T, rp)], dim=-1)
            kc.view(-1, kc.shape[-1]).index_copy_(0, kvc.slot_mapping, lat.to(kc.dtype))
            if not kvc.prefill_only:
                lora = arch.kv_lora_rank
                w_kvb = p["kv_b_proj"].view(nh_l, nope + dv, lora)
                q_lat = torch.cat([torch.einsum("thn,hnc->thc", q[..., :nope], w_kvb[:, :nope]), q_rope], dim=-1)
                if kvc.q_lens is None or q_lat.shape[0] == kvc.seq_lens.shape[0]:
                    # decode rows: one kernel reads every cached row once for all heads
                    o_lat = ops.mla_paged_decode(q_lat.contiguous(), kc, lora, kvc.block_tables, kvc.seq_lens, scale)
                else:
                    from .mla import latent_paged_attention
                    o_lat = latent_paged_attention(q_lat, kc, lora, kvc.block_tables, kvc.seq_lens, kvc.q_lens,
                                                   int(ctx.max_seqlen), scale)
                o = torch.einsum("thc,hvc->thv", o_lat.to(x.dtype), w_kvb[:, nope:])
                out = o.reshape(T, nh_l * dv)
                if partial:
                    return ctx.tp_symm.gemm_partial(out.contiguous(), p["o_proj"])
                return _row_parallel(out, p["o_proj"], ctx)
        kvb = ops.linear(c, p["kv_b_proj"]).view(T, nh_l, nope + dv)
        k_nope, v = kvb[..., :nope], kvb[..., nope:].contiguous()
        k = torch.cat([k_nope, k_rope.expand(T, nh_l, rp)], dim=-1)
        nkv_l = nh_l
        if ctx.sp is not None and ctx.sp.size > 1:
            # Ulysses: the rotary parts were rotated with this rank's positions; trade rows for heads
            q, k, v = ctx.sp.seq_to_heads(q.contiguous()), ctx.sp.seq_to_heads(k.contiguous()), ctx.sp.seq_to_heads(v)
    else:
        paged = (ctx.kv is not None and not ctx.kv.prefill_only and ctx.mrope_positions is None and not torch.is_grad_enabled()
                 and (ctx.sp is None or ctx.sp.size == 1))
        if paged and ctx.planes_ok and p.get("qkv_bias") is None and x.dim() == 2:
            qkv = ops.linear_planes(x, p["qkv"])          # the fused kernel below adds the K slices up itself
        else:
            qkv = ops.linear(x, p["qkv"], p.get("qkv_bias"))
        nkv_l = (qkv.shape[-1] // d - nh_l) // 2
        if paged:
            # steps that attend over the paged cache (decode, continuation chunks): q/k norm + RoPE and the cache
            # append are one kernel; the queries are all that comes back
            kvc = ctx.kv
            q = ops.qkv_rope_append(qkv, nh_l, nkv_l, d, p.get("q_norm"), p.get("k_norm"), arch.rms_norm_eps,
                                    ctx.attn_positions if ctx.attn_positions is not None else ctx.positions,
                                    arch.rope_theta, kvc.slot_mapping, kvc.k_cache[layer], kvc.v_cache[layer])
            o = ops.paged_attention(q, kvc.k_cache[layer], kvc.v_cache[layer], kvc.block_tables, kvc.seq_lens,
                                    kvc.q_lens, 1.0 / math.sqrt(d), groups=kvc.groups)
            if partial:
                return ctx.tp_symm.gemm_partial(o.reshape(o.shape[0], -1), p["o_proj"])
            return _row_parallel(o.reshape(o.shape[0], -1), p["o_proj"], ctx)
        q = qkv[:, :nh_l * d].view(T, nh_l, d)
        k = qkv[:, nh_l * d:(nh_l + nkv_l) * d].view(T, nkv_l, d)
        v = qkv[:, (nh_l + nkv_l) * d:].view(T, nkv_l, d)
        scale = 1.0 / math.sqrt(d)
        if ctx.sp is not None and ctx.sp.size > 1:
            # Ulysses: trade the sequence split for a head split around attention
            q, k, v = ctx.sp.seq_to_heads(q), ctx.sp.seq_to_heads(k, kv=True), ctx.sp.seq_to_heads(v, kv=True)
        if ctx.mrope_positions is not None:
            # vision-language models: time / row / column positions per rotary section
            if p.get("q_norm") is not None:
                q, k = ops.rmsnorm(q, p["q_norm"], arch.rms_norm_eps), ops.rmsnorm(k, p["k_norm"], arch.rms_norm_eps)
            q = ops.rope_mrope(q, ctx.mrope_positions, arch.rope_theta, arch.mrope_section, arch.mrope_interleaved)
            k = ops.rope_mrope(k, ctx.mrope_positions, arch.rope_theta, arch.mrope_section, arch.mrope_interleaved)
        else:
            q, k = ops.qk_norm_rope(q, k, p.get("q_norm"), p.get("k_norm"), arch.rms_norm_eps,
                                    ctx.attn_positions if ctx.attn_positions is not None else ctx.positions,
                                    arch.rope_theta)
    kv = ctx.kv
    if kv is not None:
        if not arch.use_mla:                 # (the latent row of an MLA layer is already in the cache)
            ops.kv_append(k, v, kv.k_cache[layer], kv.v_cache[layer], kv.slot_mapping)
        if kv.prefill_only:
            o = ops.attention_varlen(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, scale)
        else:
            o = ops.paged_attention(q, kv.k_cache[layer], kv.v_cache[layer], kv.block_tables,
                                    kv.seq_lens, kv.q_lens, scale, groups=kv.groups)
    elif ctx.cp is not None and ctx.cp.size > 1:
        o = ctx.cp.attention(q, k, v, ctx, scale)
    else:
        o = ops.attention_varlen(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, scale)
    if ctx.sp is not None and ctx.sp.size > 1:
        o = ctx.sp.heads_to_seq(o)
    if partial:
        return ctx.tp_symm.gemm_partial(o.reshape(o.shape[0], -1), p["o_proj"])
    out = ops.linear(o.reshape(o.shape[0], -1), p["o_proj"])
    return _tp_reduce(out, ctx)


def _tp_copy(x, ctx):
    """Input of a column-parallel layer.  Under sequence parallelism the rows are all-gathered here (the
    gradient is reduce-scattered back); otherwise identity with an all-reduce of the gradient."""
    if ctx.tp is not None and ctx.tp.size > 1:
        if ctx.seq_parallel:
            return ctx.tp.gather_sum_bwd(x)
        if torch.is_grad_enabled():
            return ctx.tp.copy_in(x)
    return x


def dense_mlp(p, x, ctx, prefix="", partial: bool = False, reduce: bool = False):
    """``reduce``: return the output already summed over the tensor-parallel group."""
    x = _tp_copy(x, ctx)
    h = ops.swiglu(ops.linear(x, p[prefix + "gate_up"]))
    if partial:
        return ctx.tp_symm.gemm_partial(h, p[prefix + "down_proj"])
    if reduce:
        return _row_parallel(h, p[prefix + "down_proj"], ctx)
    return ops.linear(h, p[prefix + "down_proj"])


def _router_aux_loss(arch: ModelArch, scores, idx, ctx: FwdCtx):
    """Load-balancing loss E · Σ_e f_e · P_e of one layer over the rows of the micro-batch.  Where the rows of a
    micro-batch are split over ranks (sequence-parallel tensor ranks, context-parallel ranks, Ulysses ranks) the
    routed fractions f and the mean probabilities P are those of all the rows: the counts are summed over the groups,
    the probability sums too, with the gradient passing to this rank's rows only (every rank adds the same loss value
    and back-propagates its own rows' share, so the ranks together apply the loss once)."""
    E, k = arch.num_experts, arch.num_experts_per_tok
    groups = []
    if ctx.seq_parallel and ctx.tp is not None and ctx.tp.size > 1:
        groups.append(ctx.tp)
    if ctx.cp is not None and ctx.cp.size > 1:
        groups.append(ctx.cp.group)
    if ctx.sp is not None and ctx.sp.size > 1:
        groups.append(ctx.sp.group)
    valid = ctx.row_valid
    if valid is not None and valid.shape[0] != scores.shape[0]:
        valid = None
    if not groups and valid is None:
        return ops.moe_aux_loss(scores, idx, E, k)
    w = torch.ones(scores.shape[0], device=scores.device) if valid is None else valid.to(torch.float32)
    f = torch.zeros(E, device=scores.device, dtype=torch.float32)
    f.index_add_(0, idx.reshape(-1), w.repeat_interleave(idx.shape[1]))
    P = (scores.float() * w[:, None]).sum(0)
    rows = w.sum()
    for g in groups:
        g.all_reduce_(f)
        g.all_reduce_(rows)
        P = g.all_reduce(P)
    rows = rows.clamp_min(1.0)
    return E * ((f / (rows * k)) * (P / rows)).sum()


def moe_block(arch: ModelArch, p, x, ctx: FwdCtx):
    logits = ops.linear(x.float(), p["router"].float())
    w, idx, scores = ops.moe_router(logits, arch.num_experts_per_tok, arch.scoring_func,
                                    arch.norm_topk_prob, p.get("router_bias"), arch.n_group,
                                    arch.topk_group, arch.routed_scaling_factor)
    if arch.router_aux_loss_coef > 0 and torch.is_grad_enabled():
        ctx.aux_losses.append(arch.router_aux_loss_coef * _router_aux_loss(arch, scores, idx, ctx))
    if p["w13"].shape[1] != 2 * arch.moe_intermediate_size:
        # expert tensor parallelism (= the TP group): every rank holds 1/tp of each expert's hidden width and
        # sees the same tokens, so its expert output is a partial sum; inputs and routing weights get their
        # gradients summed over the group, the output is all-reduced
        x_, w_ = _tp_copy(x, ctx), _tp_copy(w, ctx)
        if ctx.seq_parallel and ctx.tp is not None and ctx.tp.size > 1:
            idx = ctx.tp.all_gather_cat(idx, 0)           # the rows were gathered: so are their expert choices
        if ctx.ep is not None and ctx.ep.size > 1:
            y = ctx.ep.experts(x_, p["w13"], p["w2"], w_, idx, arch.num_experts)
        else:
            y = ops.moe_experts(x_, p["w13"], p["w2"], w_, idx)
        y = _tp_reduce(y, ctx)
    elif ctx.ep is not None and ctx.ep.size > 1:
        tp = ctx.tp
        if tp is not None and tp.size > 1 and not ctx.seq_parallel:      # (sequence-parallel rows are split already)
            # the ranks of a TP group hold the same tokens: each dispatches its own
            # 1/tp slice, so an expert sees every token once, and the outputs are
            # all-gathered back (gradient: this rank's slice)
            T = x.shape[0]
            pad = (-T) % tp.size
            # each rank back-propagates only its slice: sum the slices' gradients over TP
            x_, w_, i_ = _tp_copy(x, ctx), _tp_copy(w, ctx), idx
            if pad:
                x_, w_ = torch.nn.functional.pad(x_, (0, 0, 0, pad)), torch.nn.functional.pad(w_, (0, 0, 0, pad))
                i_ = torch.nn.functional.pad(idx, (0, 0, 0, pad))
            n = (T + pad) // tp.size
            sl = slice(tp.rank * n, (tp.rank + 1) * n)
            y_loc = ctx.ep.experts(x_[sl], p["w13"], p["w2"], w_[sl], i_[sl], arch.num_experts)
            y = tp.gather_seq(y_loc, 0)[:T]
        else:
            y = ctx.ep.experts(x, p["w13"], p["w2"], w, idx, arch.num_experts)
    else:
        y = ops.moe_experts(x, p["w13"], p["w2"], w, idx)
    if "shared_gate_up" in p:
        sh = _tp_reduce(dense_mlp(p, x, ctx, "shared_"), ctx)
        if "shared_expert_gate" in p:
            sh = sh * torch.sigmoid(torch.nn.functional.linear(x, p["shared_expert_gate"]))   # one output column
        y = y + sh
    return y


def _tp_fused_ok(p, x, ctx: FwdCtx) -> bool:
    sg = ctx.tp_symm
    return sg is not None and "router" not in p and not torch.is_grad_enabled() \
        and x.dtype == torch.bfloat16 and x.dim() == 2 and sg.fits(x.shape[0], x.shape[1])


def _decoder_layer_tp_fused(arch: ModelArch, p, x, ctx: FwdCtx, layer: int):
    """Dense layer under tensor parallelism without NCCL: the two row-parallel GEMMs
    write partial sums into symmetric staging, and one kernel per GEMM reads every
    rank's partial over NVLink, adds the residual and applies the next RMSNorm.  The
    MLP's partial stays pending in ``ctx`` and is folded into the next layer's (or the
    final) norm, so the reduced tensors never reach memory."""
    sg, eps = ctx.tp_symm, arch.rms_norm_eps
    if ctx.pending is not None:
        h = sg.ar_residual_rmsnorm(ctx.pending, x, p["input_layernorm"], eps)
        ctx.pending = None
    else:
        h = ops.rmsnorm(x, p["input_layernorm"], eps)
    a = attention_block(arch, p, h, ctx, layer, partial=True)
    h = sg.ar_residual_rmsnorm(a, x, p["post_attention_layernorm"], eps)
    ctx.pending = dense_mlp(p, h, ctx, partial=True)
    return x


def flush_pending(x, ctx: FwdCtx, norm_w=None, eps: float = 1e-6):
    """Fold a pending tensor-parallel partial into ``x``; returns ``rmsnorm(x)`` when
    ``norm_w`` is given, else ``x``."""
    part, ctx.pending = ctx.pending, None
    if torch.is_tensor(part) or hasattr(part, "planes"):   # a local sub-layer output (possibly still as K-slice planes)
        h = ops.add_rmsnorm_(x, part, norm_w, eps)
    else:
        h = ctx.tp_symm.ar_residual_rmsnorm(part, x, norm_w, eps)
    return x if norm_w is None else h


def _decoder_layer_infer_fused(arch: ModelArch, p, x, ctx: FwdCtx, layer: int):
    """Inference on CUDA without tensor-parallel partials: every residual add is fused with
    the RMSNorm that follows it (the MLP output stays pending for the next layer's norm),
    and the residual stream is updated in place."""
    eps = arch.rms_norm_eps
    # every GEMM output of this layer that goes into the residual stream is consumed by the very next kernel
    ctx.planes_ok = ctx.tp is None or ctx.tp.size == 1
    if ctx.pending is not None:
        h = flush_pending(x, ctx, p["input_layernorm"], eps)
    else:
        h = ops.rmsnorm(x, p["input_layernorm"], eps)
    a = attention_block(arch, p, h, ctx, layer)
    h = ops.add_rmsnorm_(x, a, p["post_attention_layernorm"], eps)
    ctx.pending = moe_block(arch, p, h, ctx) if "router" in p else dense_mlp(p, h, ctx, reduce=True)
    return x


def decoder_layer(arch: ModelArch, p, x, ctx: FwdCtx, layer: int):
    if arch.layer_types is not None:
        from .hybrid import hybrid_decoder_layer
        return hybrid_decoder_layer(arch, p, x, ctx, layer)
    if _tp_fused_ok(p, x, ctx):
        return _decoder_layer_tp_fused(arch, p, x, ctx, layer)
    if ctx.fuse_add_norm and not torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.bfloat16 \
            and x.dim() == 2 and x.is_contiguous():
        return _decoder_layer_infer_fused(arch, p, x, ctx, layer)
    if ctx.pending is not None:
        x = flush_pending(x, ctx)
    h = ops.rmsnorm(x, p["input_layernorm"], arch.rms_norm_eps)
    x = x + attention_block(arch, p, h, ctx, layer)
    h = ops.rmsnorm(x, p["post_attention_layernorm"], arch.rms_norm_eps)
    if "router" in p:
        return x + moe_block(arch, p, h, ctx)
    return x + dense_mlp(p, h, ctx, reduce=True)


def embed(p, tokens, ctx: FwdCtx):
    w = p["embed_tokens"]
    if ctx.tp is not None and ctx.tp.size > 1:
        Vl = w.shape[0]
        lo = ctx.tp.rank * Vl
        local = tokens - lo
        ok = (local >= 0) & (local < Vl)
        e = torch.nn.functional.embedding(local.clamp(0, Vl - 1), w)
        e = e * ok[:, None].to(e.dtype)
        return _tp_reduce(e, ctx)
    return torch.nn.functional.embedding(tokens, w)


class CausalLM:
    """Holds the parameter blocks of one model-parallel rank and runs them."""

    def __init__(self, arch: ModelArch, dtype=torch.float32, device="cpu", tp=1, tp_rank=0,
                 ep=1, ep_rank=0, layer_range=None, with_embed=True, with_head=True,
                 pad_to: int = 1, allocate: bool = True, etp: int = 1, etp_rank: int = 0):
        self.arch, self.dtype, self.device = arch, dtype, torch.device(device)
        self.tp, self.tp_rank, self.ep, self.ep_rank = tp, tp_rank, ep, ep_rank
        self.etp, self.etp_rank = etp, etp_rank
        # one (lo, hi) pair, or several when a pipeline stage holds more than one model chunk
        rs = layer_range or (0, arch.num_hidden_layers)
        self.layer_ranges = [tuple(rs)] if isinstance(rs[0], int) else [tuple(r) for r in rs]
        self.layer_range = self.layer_ranges[0]
        self.blocks: List[ParamBlock] = [
            ParamBlock(n, leaves, dtype, self.device, pad_to, allocate)
            for n, leaves in model_blocks(arch, tp, tp_rank, ep, ep_rank, layer_range,
                                          with_embed, with_head, etp, etp_rank)]
        self.block_by_name = {b.name: b for b in self.blocks}

    # ---- parameters ----
    def init_weights(self, seed: int = 1234, std: float = 0.02):
        for b in self.blocks:
            b.init_weights(seed, std)
        return self

    def num_params(self) -> int:
        return sum(lf.numel for b in self.blocks for lf in b.leaves)

    def named_leaves(self):
        for b in self.blocks:
            for lf in b.leaves:
                yield lf.name, b.params[b.short(lf.name)], lf, b

    def layer_params(self, l: int) -> Dict[str, torch.Tensor]:
        p = self.block_by_name[f"layer{l}"].params
        ex = self.block_by_name.get(f"layer{l}.experts")
        if ex is not None:
            p = {**p, **ex.params}
        return p

    def to_(self, device=None, dtype=None):
        for b in self.blocks:
            b.bind(b.flat.to(device=device or b.flat.device, dtype=dtype or b.flat.dtype))
            b.device, b.dtype = b.flat.device, b.flat.dtype
        self.device = self.blocks[0].flat.device
        self.dtype = self.blocks[0].flat.dtype
        return self

    def copy_from(self, other: "CausalLM"):
        for a, b in zip(self.blocks, other.blocks):
            a.flat.copy_(b.flat)
        return self

    # ---- forward ----
    def hidden_states(self, tokens, ctx: FwdCtx, layer_hook=None, x=None, chunk: Optional[int] = None):
        """Embedding + decoder layers (+ final norm when this rank owns the head).  ``chunk`` runs one of several
        model chunks of a pipeline stage: only the chunk that starts the model embeds, only the one that ends it
        applies the final norm."""
        lo, hi = self.layer_range if chunk is None else self.layer_ranges[chunk]
        starts = chunk is None or lo == 0
        ends = chunk is None or hi == self.arch.num_hidden_layers
        if x is None and starts and "embed" in self.block_by_name:      # a caller may supply (multimodal) input embeddings
            x = embed(self.block_by_name["embed"].params, tokens, ctx)
            if x.dtype != self.dtype:
                x = x.to(self.dtype)
        for l in range(lo, hi):
            p = self.layer_params(l)
            if layer_hook is not None:
                x = layer_hook(l, p, x, ctx)
            else:
                x = decoder_layer(self.arch, p, x, ctx, l)
            if ctx.deepstack is not None and l < len(ctx.deepstack[1]):
                # vision features of tap l join the residual stream at the image rows (a sum, so it
                # commutes with a sub-layer output that is still pending)
                rows, taps = ctx.deepstack
                x = x.index_add(0, rows, taps[l].to(x.dtype))
        if "head" in self.block_by_name and ends:
            norm_w = self.final_norm_weight()
            if ctx.pending is not None:
                return flush_pending(x, ctx, norm_w, self.arch.rms_norm_eps)
            x = ops.rmsnorm(x, norm_w, self.arch.rms_norm_eps)
        elif ctx.pending is not None:
            x = flush_pending(x, ctx)
        return x

    def final_norm_weight(self):
        w = self.block_by_name["head"].params["norm"]
        if self.arch.zero_centered_norm:
            return (1.0 + w.float()).to(w.dtype)
        return w

    def lm_head_weight(self):
        if self.arch.tie_word_embeddings:
            return self.block_by_name["embed"].params["embed_tokens"]
        return self.block_by_name["head"].params["lm_head"]

    def logits(self, hidden):
        return ops.linear(hidden, self.lm_head_weight())

    def logprobs(self, tokens, labels, ctx: FwdCtx, temperature=1.0, layer_hook=None, x=None):
        """Per-token log p(label) and entropy for a packed row, never building ``[T, V]``.
        ``x``: input embeddings to use instead of the token embeddings (multimodal rows)."""
        h = self.hidden_states(tokens, ctx, layer_hook, x=x)
        w = self.lm_head_weight()
        if ctx.tp is not None and ctx.tp.size > 1 and w.shape[0] != self.arch.vocab_size:
            from chatlearn_b200.parallel.tp_ops import vocab_parallel_logprob_entropy
            return vocab_parallel_logprob_entropy(h, w, labels, ctx.tp, temperature)
        return ops.lmhead_logprob_entropy(h, w, labels, temperature)

    def score(self, tokens, ctx: FwdCtx):
        """Reward/value head: ``[T, num_labels]``."""
        h = self.hidden_states(tokens, ctx)
        return ops.linear(h, self.block_by_name["head"].params["score"]).float()

    # ---- HF state dict ----
    @torch.no_grad()
    def hf_state_dict(self, dtype=None) -> Dict[str, torch.Tensor]:
        """Assemble full HF tensors from this rank's leaves (complete only when
        tp == ep == 1 and all layers are local; otherwise partial tensors of the
        local shard are returned under the same names)."""
        out: Dict[str, torch.Tensor] = {}
        one_d = set()
        for _, p, lf, _ in self.named_leaves():
            for s in lf.segments:
                if len(lf.shape) == 1:
                    one_d.add(s.hf_name)
                full = out.get(s.hf_name)
                if full is None:
                    full = torch.zeros(s.hf_shape, dtype=dtype or p.dtype, device=p.device)
                    out[s.hf_name] = full
                slab = p if len(lf.shape) < 3 else p[s.dst_index]
                slab = slab.reshape(lf.matrix_shape)
                r0, c0 = s.dst_start
                rs, cs = s.src_start
                nr, nc = s.extent
                full[rs:rs + nr, cs:cs + nc] = slab[r0:r0 + nr, c0:c0 + nc]
        for k in one_d:
            out[k] = out[k].squeeze(1)
        for k in list(out):
            if k.endswith(".conv1d.weight"):        # depthwise Conv1d weights are [channels, 1, taps]
                out[k] = out[k].unsqueeze(1)
        for k, shape in getattr(self, "hf_reshape", {}).items():
            if k in out:                            # e.g. the vision tower's patch-embedding convolution kernel
                out[k] = out[k].reshape(shape)
        return out

    @torch.no_grad()
    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True):
        """Fill the local leaves from full HF tensors (each rank slices its shard)."""
        missing = []
        for _, p, lf, _ in self.named_leaves():
            for s in lf.segments:
                src = sd.get(s.hf_name)
                if src is None:
                    missing.append(s.hf_name)
                    continue
                src = src.reshape(s.hf_shape)
                slab = p if len(lf.shape) < 3 else p[s.dst_index]
                slab = slab.view(lf.matrix_shape)
                r0, c0 = s.dst_start
                rs, cs = s.src_start
                nr, nc = s.extent
                slab[r0:r0 + nr, c0:c0 + nc].copy_(src[rs:rs + nr, cs:cs + nc])
        if strict and missing:
            raise KeyError(f"missing tensors: {sorted(set(missing))[:8]} …")
        return missing


def packed_ctx(seq_lens: List[int], device, **kw) -> Tuple[FwdCtx, torch.Tensor]:
    """Context of a packed row made of sequences of the given lengths."""
    cu = torch.zeros(len(seq_lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(seq_lens, dtype=torch.int32).cumsum(0)
    pos = torch.cat([torch.arange(n) for n in seq_lens]) if seq_lens else torch.zeros(0, dtype=torch.long)
    ctx = FwdCtx(positions=pos.to(device), cu_seqlens=cu.to(device),
                 max_seqlen=max(seq_lens) if seq_lens else 0, **kw)
    return ctx, cu
