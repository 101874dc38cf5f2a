"""Qwen3-Next layers: gated delta-net token mixers with a recurrent state, interleaved with
gated softmax attention (a quarter of each head rotates, the output is scaled by a sigmoid
gate that q_proj emits beside the query), zero-centred RMSNorm and an MoE with one
sigmoid-gated shared expert.

The reference trains this family through HF/Megatron modules and patches only its MoE block
(chatlearn/models/patches/transformers/qwen3_next_moe_patch.py:41-85); its Megatron weight
mapping is chatlearn/synchronizer/mappers/megatron_llm_mapper.py:262-343.  Here the layers are
functions over the flat parameter blocks like every other family.  The delta rule runs
chunk-wise on PyTorch statements (one batched triangular solve per chunk instead of a
token-by-token scan) for training and prefill, and as a single recurrent update per decoded
token; packed rows are scattered into a padded [sequences, longest] batch first, with padded
positions made neutral (no decay, no write) so the final state of every sequence is exact.
"""
import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F

from chatlearn_b200 import ops
from .arch import ModelArch

CHUNK = 64


@dataclass
class LinearState:
    """Per-sequence state of the gated delta-net layers in the rollout engine."""
    conv: List[Optional[torch.Tensor]]     # per layer [state slots, taps - 1, channels]
    rec: List[Optional[torch.Tensor]]      # per layer [state slots, value heads, dk, dv] fp32
    slots: torch.Tensor                    # [B] state slot of every sequence of this step
    fresh: torch.Tensor                    # [B] bool: the sequence starts at position 0 (state is zero)


def zc(w: torch.Tensor) -> torch.Tensor:
    """Scale vector of a zero-centred RMSNorm."""
    return (1.0 + w.float()).to(w.dtype)


def _l2norm(x, eps=1e-6):
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gated_delta_chunked(q, k, v, g, beta, init=None, chunk: int = CHUNK):
    """Gated delta rule ``S_t = a_t S_{t-1} + k_t^T b_t (v_t - k_t a_t S_{t-1})``, ``o_t = q_t S_t``
    with ``a_t = exp(g_t)``, evaluated chunk by chunk.  ``q, k``: [B, L, H, dk] (normalised, q scaled),
    ``v``: [B, L, H, dv], ``g, beta``: [B, L, H]; everything fp32.  Returns ``(o [B, L, H, dv], S [B, H, dk, dv])``.

    Inside a chunk with cumulative log-decay c: the writes solve ``(I + A) X = [b v | b k e^c]`` where
    ``A`` is the strictly lower part of ``(b k) k^T * e^{c_i - c_j}`` — one unit-triangular solve."""
    B, L, H, dk = q.shape
    dv = v.shape[-1]
    pad = (-L) % chunk
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = F.pad(g, (0, 0, 0, pad)), F.pad(beta, (0, 0, 0, pad))
    n = (L + pad) // chunk
    q, k, v = (t.permute(0, 2, 1, 3).reshape(B, H, n, chunk, t.shape[-1]) for t in (q, k, v))
    c = g.permute(0, 2, 1).reshape(B, H, n, chunk).cumsum(-1)
    b = beta.permute(0, 2, 1).reshape(B, H, n, chunk, 1)
    kb, vb = k * b, v * b
    lower = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril()
    diff = (c.unsqueeze(-1) - c.unsqueeze(-2)).masked_fill(~lower, float("-inf"))
    decay = diff.exp()                                                  # e^{c_i - c_j} for j <= i, else 0
    A = (kb @ k.transpose(-1, -2)) * decay                              # the solve ignores its diagonal
    rhs = torch.cat([vb, kb * c.exp().unsqueeze(-1)], dim=-1)
    X = torch.linalg.solve_triangular(A, rhs, upper=False, unitriangular=True)
    U, W = X[..., :dv], X[..., dv:]
    qk = (q @ k.transpose(-1, -2)) * decay
    S = q.new_zeros(B, H, dk, dv) if init is None else init.to(q.dtype)
    outs = []
    for i in range(n):
        ci = c[:, :, i]
        v_new = U[:, :, i] - W[:, :, i] @ S
        outs.append((q[:, :, i] * ci.exp().unsqueeze(-1)) @ S + qk[:, :, i] @ v_new)
        tail = (ci[..., -1:] - ci).exp().unsqueeze(-1)                   # decay from each position to the chunk end
        S = S * ci[..., -1].exp()[..., None, None] + (k[:, :, i] * tail).transpose(-1, -2) @ v_new
    o = torch.stack(outs, 2).reshape(B, H, n * chunk, dv)[:, :, :L].permute(0, 2, 1, 3)
    return o, S


def gated_delta_step(q, k, v, g, beta, S):
    """One token per sequence: ``q, k`` [B, H, dk], ``v`` [B, H, dv], ``g, beta`` [B, H], ``S`` [B, H, dk, dv]."""
    S = S * g.exp()[..., None, None]
    mem = (S * k.unsqueeze(-1)).sum(-2)
    S = S + k.unsqueeze(-1) * ((v - mem) * beta.unsqueeze(-1)).unsqueeze(-2)
    return (S * q.unsqueeze(-1)).sum(-2), S


def _pack_index(ctx, T: int, device):
    """Row -> (sequence, offset) of a packed row; ``(seq, off, B, L, lens)``."""
    if ctx.cu_seqlens is None:
        ar = torch.arange(T, device=device)
        return ar, torch.zeros_like(ar), T, 1, torch.ones_like(ar)
    cu = ctx.cu_seqlens.long()
    B = cu.numel() - 1
    lens = cu[1:] - cu[:-1]
    seq = torch.repeat_interleave(torch.arange(B, device=device), lens, output_size=T)
    off = torch.arange(T, device=device) - cu[seq]
    return seq, off, B, int(ctx.max_seqlen), lens


class _HeadExchange:
    """Rows of all heads <-> all rows of 1/n of the heads, over the Ulysses group or the context-parallel group.  A
    context-parallel rank holds a zig-zag slice of every sequence: after the exchange the rows arrive rank by rank and
    are put back into sequence order (``inv``), and leave in rank order again (``fwd``)."""

    def __init__(self, ctx):
        from chatlearn_b200.parallel.ulysses import UlyssesGroup
        self.inv = self.fwd = None
        if ctx.sp is not None and ctx.sp.size > 1:
            self.ex = ctx.sp
        else:
            self.ex = UlyssesGroup(ctx.cp.group)
            self.inv = ctx.cp_plan["inv"]
            self.fwd = torch.empty_like(self.inv)
            self.fwd[self.inv] = torch.arange(self.inv.numel(), device=self.inv.device)
        self.size, self.rank = self.ex.size, self.ex.rank

    @staticmethod
    def of(ctx):
        if (ctx.sp is not None and ctx.sp.size > 1) or (ctx.cp is not None and ctx.cp.size > 1):
            return _HeadExchange(ctx)
        return None

    def seq_to_heads(self, x):
        y = self.ex.seq_to_heads(x)
        return y if self.inv is None else y.index_select(0, self.inv)

    def heads_to_seq(self, x):
        return self.ex.heads_to_seq(x.contiguous() if self.fwd is None else x.index_select(0, self.fwd))


def gated_delta_net(arch: ModelArch, p, x, ctx, layer: int):
    T = x.shape[0]
    if T == 0:
        return x
    from .model import _tp_copy
    x = _tp_copy(x, ctx)                       # (sequence-parallel rows are gathered here)
    T = x.shape[0]
    dk, dv, K = arch.linear_key_head_dim, arch.linear_value_head_dim, arch.linear_conv_kernel_dim
    r = arch.linear_num_value_heads // arch.linear_num_key_heads
    nv = p["A_log"].shape[0]                   # this rank's heads (1/tp of the layer's)
    nk = nv // r
    kd, vd = nk * dk, nv * dv
    C = 2 * kd + vd
    st: Optional[LinearState] = ctx.kv.lin if ctx.kv is not None else None
    proj = ops.linear(x, p["in_proj"])
    pq = 2 * kd + 2 * vd
    qkvz = proj[:, :pq].view(T, nk, 2 * dk + 2 * r * dv)
    ba = proj[:, pq:].view(T, nk, 2 * r)
    z = qkvz[..., 2 * dk + r * dv:].reshape(T, nv, dv)
    mixed = torch.cat([qkvz[..., :dk].reshape(T, kd), qkvz[..., dk:2 * dk].reshape(T, kd),
                       qkvz[..., 2 * dk:2 * dk + r * dv].reshape(T, vd)], dim=-1)
    bgate = torch.sigmoid(ba[..., :r].reshape(T, nv).float())
    g = -p["A_log"].float().exp() * F.softplus(ba[..., r:].reshape(T, nv).float() + p["dt_bias"].float())
    conv_w = p["conv1d"]
    sp = _HeadExchange.of(ctx)
    if sp is not None:
        # Ulysses / context parallelism: trade the sequence split for a head split around the convolution and the
        # recurrence (both run per head over whole sequences): this rank gets 1/n of the key heads with their value
        # heads, all rows
        assert st is None and nk % sp.size == 0, \
            "sequence-split delta-net layers need the key heads divisible by the group, and no rollout state"
        T_loc, nv_all, vd_all = T, nv, vd
        q_ = sp.seq_to_heads(mixed[:, :kd].reshape(T, nk, dk))
        k_ = sp.seq_to_heads(mixed[:, kd:2 * kd].reshape(T, nk, dk))
        v_ = sp.seq_to_heads(mixed[:, 2 * kd:].reshape(T, nv, dv))
        gb = sp.seq_to_heads(torch.stack([g, bgate], dim=-1))
        nk_l, nv_l = nk // sp.size, nv // sp.size
        lo_k, lo_v = sp.rank * nk_l * dk, sp.rank * nv_l * dv
        conv_w = torch.cat([conv_w.narrow(0, lo_k, nk_l * dk), conv_w.narrow(0, kd + lo_k, nk_l * dk),
                            conv_w.narrow(0, 2 * kd + lo_v, nv_l * dv)], dim=0)
        nk, nv, T = nk_l, nv_l, q_.shape[0]
        kd, vd = nk * dk, nv * dv
        C = 2 * kd + vd
        mixed = torch.cat([q_.reshape(T, kd), k_.reshape(T, kd), v_.reshape(T, vd)], dim=-1)
        g, bgate = gb[..., 0].contiguous(), gb[..., 1].contiguous()

    seq, off, B, L, lens = _pack_index(ctx, T, x.device)
    # causal depthwise convolution over [previous taps | this step's rows] of every sequence
    xp = mixed.new_zeros(B, L + K - 1, C)
    if st is not None:
        keep = (~st.fresh).to(mixed.dtype)[:, None, None]
        xp[:, :K - 1] = st.conv[layer].index_select(0, st.slots).to(mixed.dtype) * keep
    xp[seq, off + K - 1] = mixed
    if L == 1:
        # decode: one output per channel, the taps times the last K inputs (plain statements, safe to capture)
        y = F.silu((xp.float() * conv_w.float().t().unsqueeze(0)).sum(1, keepdim=True)).to(mixed.dtype)
    else:
        y = F.silu(F.conv1d(xp.transpose(1, 2), conv_w.unsqueeze(1).to(mixed.dtype), groups=C)).transpose(1, 2)
    if st is not None:
        idx = (lens[:, None] + torch.arange(K - 1, device=x.device)[None]).unsqueeze(-1).expand(B, K - 1, C)
        st.conv[layer].index_copy_(0, st.slots, xp.gather(1, idx).to(st.conv[layer].dtype))
    if L == 1 and T == B and st is not None and x.is_cuda and not torch.is_grad_enabled() and ops.get_mode() == "native":
        # decode on the GPU: normalisation, grouped heads, decay, write and read-out of the state in one kernel
        from chatlearn_b200.ops import native
        y1 = y[:, 0]
        o = native.C.gdn_decode_step(y1[:, :kd].reshape(B, nk, dk).contiguous(), y1[:, kd:2 * kd].reshape(B, nk, dk).contiguous(),
                                     y1[:, 2 * kd:].reshape(B, nv, dv).contiguous(), g.contiguous(), bgate.contiguous(),
                                     st.rec[layer], st.slots, st.fresh, 1.0 / math.sqrt(dk))
        native.launch_counts["gdn_decode_step"] += 1
        return _gdn_output(arch, p, o, z, x.dtype, T, vd, ctx)
    q = _l2norm(y[..., :kd].reshape(B, L, nk, dk).float()) * (1.0 / math.sqrt(dk))
    k = _l2norm(y[..., kd:2 * kd].reshape(B, L, nk, dk).float())
    v = y[..., 2 * kd:].reshape(B, L, nv, dv).float()
    if r > 1:
        q, k = q.repeat_interleave(r, dim=2), k.repeat_interleave(r, dim=2)
    # padded positions neither decay nor write
    gp, bp = g.new_zeros(B, L, nv), bgate.new_zeros(B, L, nv)
    gp[seq, off], bp[seq, off] = g, bgate
    init = None
    if st is not None:
        init = st.rec[layer].index_select(0, st.slots) * (~st.fresh).float()[:, None, None, None]
    if L == 1:
        o, S = gated_delta_step(q[:, 0], k[:, 0], v[:, 0], gp[:, 0], bp[:, 0],
                                init if init is not None else q.new_zeros(B, nv, dk, dv))
        o = o.unsqueeze(1)
    else:
        o, S = gated_delta_chunked(q, k, v, gp, bp, init)
    if st is not None:
        st.rec[layer].index_copy_(0, st.slots, S.to(st.rec[layer].dtype))
    o = o[seq, off]                                                        # back to the packed row: [T, nv, dv]
    if sp is not None:
        o = sp.heads_to_seq(o)                                             # this rank's rows, all heads
        T, vd = T_loc, vd_all
    return _gdn_output(arch, p, o, z, x.dtype, T, vd, ctx)


def _gdn_output(arch, p, o, z, dtype, T, vd, ctx):
    """Per-head RMSNorm of the read-out, gated by silu(z), then the (row-parallel) output projection."""
    from .model import _row_parallel
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + arch.rms_norm_eps)
    o = (p["gdn_norm"] * o.to(dtype)).float() * F.silu(z.float())
    return _row_parallel(o.to(dtype).reshape(T, vd), p["out_proj"], ctx)


def gated_attention(arch: ModelArch, p, x, ctx, layer: int):
    from .model import _row_parallel, _tp_copy
    sp = ctx.sp if ctx.sp is not None and ctx.sp.size > 1 else None
    x = _tp_copy(x, ctx)
    T = x.shape[0]
    d = arch.head_dim
    nh = p["o_proj"].shape[1] // d             # this rank's query heads and key/value heads
    nkv = (p["qkv"].shape[0] // d - 2 * nh) // 2
    qkv = ops.linear(x, p["qkv"])
    qg = qkv[:, :2 * nh * d].view(T, nh, 2 * d)
    q, gate = qg[..., :d], qg[..., d:].reshape(T, nh * d)
    k = qkv[:, 2 * nh * d:(2 * nh + nkv) * d].view(T, nkv, d)
    v = qkv[:, (2 * nh + nkv) * d:].view(T, nkv, d)
    q = ops.rmsnorm(q.contiguous(), zc(p["q_norm"]), arch.rms_norm_eps)
    k = ops.rmsnorm(k.contiguous(), zc(p["k_norm"]), arch.rms_norm_eps)
    rd = arch.rotary_dim
    if rd > 0 and T > 0:
        pos = ctx.positions
        q = torch.cat([ops.rope(q[..., :rd].contiguous(), pos, arch.rope_theta), q[..., rd:]], dim=-1)
        k = torch.cat([ops.rope(k[..., :rd].contiguous(), pos, arch.rope_theta), k[..., rd:]], dim=-1)
    scale = 1.0 / math.sqrt(d)
    kv = ctx.kv
    if sp is not None:
        # Ulysses: all rows of 1/sp of the heads through attention, then back (the output gate stays with the rows)
        assert kv is None
        q, k, v = sp.seq_to_heads(q.contiguous()), sp.seq_to_heads(k.contiguous(), kv=True), sp.seq_to_heads(v.contiguous(), kv=True)
    if kv is not None:
        ops.kv_append(k, v.contiguous(), kv.k_cache[layer], kv.v_cache[layer], kv.slot_mapping)
        if kv.prefill_only:
            o = ops.attention_varlen(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, scale)
        else:
            o = ops.paged_attention(q, kv.k_cache[layer], kv.v_cache[layer], kv.block_tables,
                                    kv.seq_lens, kv.q_lens, scale)
    elif ctx.cp is not None and ctx.cp.size > 1:
        o = ctx.cp.attention(q.contiguous(), k.contiguous(), v.contiguous(), ctx, scale)    # keys / values gathered
    else:
        o = ops.attention_varlen(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, scale)
    if sp is not None:
        o = sp.heads_to_seq(o.contiguous())
    o = o.reshape(T, nh * d) * torch.sigmoid(gate)
    return _row_parallel(o, p["o_proj"], ctx)


def hybrid_decoder_layer(arch: ModelArch, p, x, ctx, layer: int):
    from .model import dense_mlp, flush_pending, moe_block
    if ctx.pending is not None:
        x = flush_pending(x, ctx)
    eps = arch.rms_norm_eps
    h = ops.rmsnorm(x, zc(p["input_layernorm"]), eps)
    mix = gated_delta_net(arch, p, h, ctx, layer) if "in_proj" in p else gated_attention(arch, p, h, ctx, layer)
    x = x + mix
    h = ops.rmsnorm(x, zc(p["post_attention_layernorm"]), eps)
    return x + (moe_block(arch, p, h, ctx) if "router" in p else dense_mlp(p, h, ctx, reduce=True))
