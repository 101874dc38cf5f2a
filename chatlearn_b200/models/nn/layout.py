"""Parameter layout: how a model instance's local tensors ("leaves") map onto the
canonical HuggingFace tensors.

Every model instance — FSDP-style trainer, TP/EP-sharded trainer, rollout
engine — stores fused leaves (``qkv``, ``gate_up``, stacked expert ``w13``/``w2``)
holding only its own shard.  A leaf is described by a list of ``Segment``s, each
saying "this rectangle of the leaf is that rectangle of HF tensor X".  The HF
coordinate space is the common language: checkpoints read/write through it, and
the trainer→rollout synchronizer intersects source and destination segments in
it to obtain copy descriptors.  This replaces the reference's per-engine
mappers and ``ShardedTensorInfo`` algebra
(chatlearn/synchronizer/mappers/*.py, chatlearn/utils/mappings/sharded_tensor_info.py)
with one declarative table; QKV packing, gate/up packing, GQA replication and
expert re-homing fall out of the segment lists.
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from .arch import ModelArch


@dataclass(frozen=True)
class Segment:
    hf_name: str
    hf_shape: Tuple[int, int]          # full HF tensor as 2-D (1-D tensors are (n, 1))
    src_start: Tuple[int, int]         # (row, col) in the HF tensor
    extent: Tuple[int, int]            # (rows, cols)
    dst_start: Tuple[int, int]         # (row, col) inside the leaf matrix
    dst_index: int = 0                 # leading index for 3-D leaves (local expert id)


@dataclass
class Leaf:
    name: str                          # local name, e.g. "layers.3.qkv"
    shape: Tuple[int, ...]             # local shape (1-D, 2-D or 3-D [n, rows, cols])
    init: str = "normal"               # normal | ones | zeros
    segments: List[Segment] = field(default_factory=list)
    replicated: bool = False           # same content on every model-parallel rank
    grad_sum_tp: bool = False          # gradient is a partial sum per TP rank (needs an all-reduce)
    # key/value heads replicated over tensor-parallel ranks (tp > kv heads): (first row, rows, this rank's kv head,
    # kv heads); the gradients of those rows are summed over the ranks that hold the same head
    grad_sum_kv: Optional[Tuple[int, int, int, int]] = None

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def matrix_shape(self) -> Tuple[int, int]:
        """(rows, cols) of one 2-D slab of the leaf."""
        if len(self.shape) == 1:
            return (self.shape[0], 1)
        return (self.shape[-2], self.shape[-1])


def _full(leaf_name, shape, hf_name, init="normal", replicated=True) -> Leaf:
    ms = (shape[0], 1) if len(shape) == 1 else tuple(shape)
    return Leaf(leaf_name, tuple(shape), init,
                [Segment(hf_name, ms, (0, 0), ms, (0, 0))], replicated)


def _rows(hf_name, full_shape, r0, n, dst_row, dst_index=0):
    return Segment(hf_name, full_shape, (r0, 0), (n, full_shape[1]), (dst_row, 0), dst_index)


def _cols(hf_name, full_shape, c0, n, dst_col=0, dst_index=0):
    return Segment(hf_name, full_shape, (0, c0), (full_shape[0], n), (0, dst_col), dst_index)


def kv_head_range(arch: ModelArch, tp: int, tp_rank: int) -> Tuple[int, int]:
    """(first kv head, count) owned by a TP rank; heads are replicated when tp > n_kv."""
    nkv = arch.num_key_value_heads
    if tp <= nkv:
        assert nkv % tp == 0, f"{nkv} kv heads not divisible by tp={tp}"
        per = nkv // tp
        return tp_rank * per, per
    assert tp % nkv == 0, f"tp={tp} must be a multiple of {nkv} kv heads"
    return tp_rank // (tp // nkv), 1


def _hybrid_mixer_leaves(arch: ModelArch, l: int, pre: str, hp: str, tp: int = 1, tp_rank: int = 0) -> List[Leaf]:
    """Token mixer of a Qwen3-Next layer (HF names: transformers
    models/qwen3_next/modeling_qwen3_next.py, ``Qwen3NextGatedDeltaNet`` / ``Qwen3NextAttention``; the
    reference maps the same tensors for Megatron in
    chatlearn/synchronizer/mappers/megatron_llm_mapper.py:262-343).  Under tensor parallelism a rank owns
    ``1/tp`` of the key heads of a delta-net layer with their value heads (input projections, convolution
    channels, decay parameters by rows; output projection by columns) and ``1/tp`` of the query heads of a gated
    attention layer with their output gates."""
    H = arch.hidden_size
    if arch.layer_is_linear(l):
        a = hp + "linear_attn."
        nk, nv = arch.linear_num_key_heads, arch.linear_num_value_heads
        dk, dv = arch.linear_key_head_dim, arch.linear_value_head_dim
        assert nk % tp == 0, f"{nk} key heads of the delta-net layers not divisible by tp={tp}"
        nk_l, nv_l = nk // tp, nv // tp
        kd, vd = nk * dk, nv * dv
        kd_l, vd_l = nk_l * dk, nv_l * dv
        pq, pq_l = 2 * kd + 2 * vd, 2 * kd_l + 2 * vd_l
        C, K = 2 * kd + vd, arch.linear_conv_kernel_dim
        # one GEMM for both input projections: rows [q k v z per key-head group | b a per group]
        in_proj = Leaf(pre + "in_proj", (pq_l + 2 * nv_l, H), "normal",
                       [_rows(a + "in_proj_qkvz.weight", (pq, H), tp_rank * pq_l, pq_l, 0),
                        _rows(a + "in_proj_ba.weight", (2 * nv, H), tp_rank * 2 * nv_l, 2 * nv_l, pq_l)])
        if tp == 1:
            conv = _full(pre + "conv1d", (C, K), a + "conv1d.weight", "conv")
            dt_bias = _full(pre + "dt_bias", (nv,), a + "dt_bias", "ones")
            a_log = _full(pre + "A_log", (nv,), a + "A_log", "a_log")
            out_proj = _full(pre + "out_proj", (H, vd), a + "out_proj.weight")
        else:
            # channels of the convolution: [q | k | v], each split by heads
            conv = Leaf(pre + "conv1d", (2 * kd_l + vd_l, K), "conv",
                        [_rows(a + "conv1d.weight", (C, K), tp_rank * kd_l, kd_l, 0),
                         _rows(a + "conv1d.weight", (C, K), kd + tp_rank * kd_l, kd_l, kd_l),
                         _rows(a + "conv1d.weight", (C, K), 2 * kd + tp_rank * vd_l, vd_l, 2 * kd_l)])
            dt_bias = Leaf(pre + "dt_bias", (nv_l,), "ones", [_rows(a + "dt_bias", (nv, 1), tp_rank * nv_l, nv_l, 0)])
            a_log = Leaf(pre + "A_log", (nv_l,), "a_log", [_rows(a + "A_log", (nv, 1), tp_rank * nv_l, nv_l, 0)])
            out_proj = Leaf(pre + "out_proj", (H, vd_l), "normal",
                            [_cols(a + "out_proj.weight", (H, vd), tp_rank * vd_l, vd_l)])
        norm = _full(pre + "gdn_norm", (dv,), a + "norm.weight", "ones")
        norm.grad_sum_tp = tp > 1                 # shared by all heads: every rank holds a partial gradient
        return [in_proj, conv, dt_bias, a_log, norm, out_proj]
    a = hp + "self_attn."
    nh, nkv, d = arch.num_attention_heads, arch.num_key_value_heads, arch.head_dim
    nh_l = nh // tp
    kv0, nkv_l = kv_head_range(arch, tp, tp_rank)
    qf, kf = (nh * 2 * d, H), (nkv * d, H)       # q_proj rows per head: [query | gate]
    qkv = Leaf(pre + "qkv", ((2 * nh_l + 2 * nkv_l) * d, H), "normal",
               [_rows(a + "q_proj.weight", qf, tp_rank * nh_l * 2 * d, nh_l * 2 * d, 0),
                _rows(a + "k_proj.weight", kf, kv0 * d, nkv_l * d, nh_l * 2 * d),
                _rows(a + "v_proj.weight", kf, kv0 * d, nkv_l * d, (2 * nh_l + nkv_l) * d)])
    if tp > nkv:
        qkv.grad_sum_kv = (2 * nh_l * d, 2 * nkv_l * d, kv0, nkv)
    qn = _full(pre + "q_norm", (d,), a + "q_norm.weight", "zeros")
    kn = _full(pre + "k_norm", (d,), a + "k_norm.weight", "zeros")
    qn.grad_sum_tp = kn.grad_sum_tp = tp > 1
    o_proj = Leaf(pre + "o_proj", (H, nh_l * d), "normal",
                  [_cols(a + "o_proj.weight", (H, nh * d), tp_rank * nh_l * d, nh_l * d)])
    return [qkv, qn, kn, o_proj]


def layer_leaves(arch: ModelArch, l: int, tp: int = 1, tp_rank: int = 0, ep: int = 1,
                 ep_rank: int = 0, etp: int = 1, etp_rank: int = 0) -> List[Leaf]:
    """Leaves of decoder layer ``l`` for one (tp, ep) rank."""
    H = arch.hidden_size
    pre, hp = f"layers.{l}.", f"model.layers.{l}."
    norm_init = "zeros" if arch.zero_centered_norm else "ones"      # zero-centred norms scale by (1 + w)
    out: List[Leaf] = [_full(pre + "input_layernorm", (H,), hp + "input_layernorm.weight", norm_init)]
    nh = arch.num_attention_heads
    assert nh % tp == 0, f"{nh} heads not divisible by tp={tp}"
    nh_l = nh // tp
    if arch.layer_types is not None:
        out.extend(_hybrid_mixer_leaves(arch, l, pre, hp, tp, tp_rank))
    elif arch.use_mla:
        qd = arch.qk_nope_head_dim + arch.qk_rope_head_dim
        a = hp + "self_attn."
        if arch.q_lora_rank:
            out.append(_full(pre + "q_a_proj", (arch.q_lora_rank, H), a + "q_a_proj.weight"))
            out.append(_full(pre + "q_a_layernorm", (arch.q_lora_rank,), a + "q_a_layernorm.weight", "ones"))
            # the compressed query feeds this rank's heads only: the gradients of the two are partial sums
            out[-1].grad_sum_tp = out[-2].grad_sum_tp = tp > 1
            fs = (nh * qd, arch.q_lora_rank)
            out.append(Leaf(pre + "q_b_proj", (nh_l * qd, arch.q_lora_rank), "normal",
                            [_rows(a + "q_b_proj.weight", fs, tp_rank * nh_l * qd, nh_l * qd, 0)]))
        else:
            fs = (nh * qd, H)
            out.append(Leaf(pre + "q_proj", (nh_l * qd, H), "normal",
                            [_rows(a + "q_proj.weight", fs, tp_rank * nh_l * qd, nh_l * qd, 0)]))
        out.append(_full(pre + "kv_a_proj_with_mqa", (arch.kv_lora_rank + arch.qk_rope_head_dim, H),
                         a + "kv_a_proj_with_mqa.weight"))
        out.append(_full(pre + "kv_a_layernorm", (arch.kv_lora_rank,), a + "kv_a_layernorm.weight", "ones"))
        # the latent and the rotary key are shared by all heads, of which a rank sees its own: partial gradients
        out[-1].grad_sum_tp = out[-2].grad_sum_tp = tp > 1
        kvd = arch.qk_nope_head_dim + arch.v_head_dim
        fs = (nh * kvd, arch.kv_lora_rank)
        out.append(Leaf(pre + "kv_b_proj", (nh_l * kvd, arch.kv_lora_rank), "normal",
                        [_rows(a + "kv_b_proj.weight", fs, tp_rank * nh_l * kvd, nh_l * kvd, 0)]))
        fs = (H, nh * arch.v_head_dim)
        out.append(Leaf(pre + "o_proj", (H, nh_l * arch.v_head_dim), "normal",
                        [_cols(a + "o_proj.weight", fs, tp_rank * nh_l * arch.v_head_dim,
                               nh_l * arch.v_head_dim)]))
    else:
        d = arch.head_dim
        kv0, nkv_l = kv_head_range(arch, tp, tp_rank)
        a = hp + "self_attn."
        qf, kf = (nh * d, H), (arch.num_key_value_heads * d, H)
        segs = [_rows(a + "q_proj.weight", qf, tp_rank * nh_l * d, nh_l * d, 0),
                _rows(a + "k_proj.weight", kf, kv0 * d, nkv_l * d, nh_l * d),
                _rows(a + "v_proj.weight", kf, kv0 * d, nkv_l * d, (nh_l + nkv_l) * d)]
        rows = (nh_l + 2 * nkv_l) * d
        out.append(Leaf(pre + "qkv", (rows, H), "normal", segs))
        kv_rep = (nh_l * d, 2 * nkv_l * d, kv0, arch.num_key_value_heads) if tp > arch.num_key_value_heads else None
        out[-1].grad_sum_kv = kv_rep
        if arch.attention_bias:
            bs = [Segment(a + "q_proj.bias", (nh * d, 1), (tp_rank * nh_l * d, 0), (nh_l * d, 1), (0, 0)),
                  Segment(a + "k_proj.bias", (kf[0], 1), (kv0 * d, 0), (nkv_l * d, 1), (nh_l * d, 0)),
                  Segment(a + "v_proj.bias", (kf[0], 1), (kv0 * d, 0), (nkv_l * d, 1), ((nh_l + nkv_l) * d, 0))]
            out.append(Leaf(pre + "qkv_bias", (rows,), "zeros", bs))
            out[-1].grad_sum_kv = kv_rep
        if arch.qk_norm:
            out.append(_full(pre + "q_norm", (d,), a + "q_norm.weight", "ones"))
            out.append(_full(pre + "k_norm", (d,), a + "k_norm.weight", "ones"))
            # shared by all heads: with heads split over TP each rank sees a partial gradient
            out[-1].grad_sum_tp = out[-2].grad_sum_tp = tp > 1
        fs = (H, nh * d)
        out.append(Leaf(pre + "o_proj", (H, nh_l * d), "normal",
                        [_cols(a + "o_proj.weight", fs, tp_rank * nh_l * d, nh_l * d)]))
    out.append(_full(pre + "post_attention_layernorm", (H,), hp + "post_attention_layernorm.weight", norm_init))

    def mlp_leaves(prefix, hf_prefix, F, shard_tp):
        t, r = (tp, tp_rank) if shard_tp else (1, 0)
        assert F % t == 0
        Fl = F // t
        gu = Leaf(prefix + "gate_up", (2 * Fl, H), "normal",
                  [_rows(hf_prefix + "gate_proj.weight", (F, H), r * Fl, Fl, 0),
                   _rows(hf_prefix + "up_proj.weight", (F, H), r * Fl, Fl, Fl)])
        dn = Leaf(prefix + "down_proj", (H, Fl), "normal",
                  [_cols(hf_prefix + "down_proj.weight", (H, F), r * Fl, Fl)])
        return [gu, dn]

    if arch.layer_is_moe(l):
        E, Fm = arch.num_experts, arch.moe_intermediate_size
        assert E % ep == 0, f"{E} experts not divisible by ep={ep}"
        El = E // ep
        assert Fm % etp == 0, f"expert width {Fm} not divisible by etp={etp}"
        Fe = Fm // etp
        m = hp + "mlp."
        out.append(_full(pre + "router", (E, H), m + "gate.weight"))
        if arch.router_bias:
            out.append(_full(pre + "router_bias", (E,), m + "gate.e_score_correction_bias", "zeros"))
        s13, s2 = [], []
        for j in range(El):
            e = ep_rank * El + j
            # expert tensor parallelism: every rank of the group keeps 1/etp of each expert's hidden width
            s13.append(_rows(f"{m}experts.{e}.gate_proj.weight", (Fm, H), etp_rank * Fe, Fe, 0, j))
            s13.append(_rows(f"{m}experts.{e}.up_proj.weight", (Fm, H), etp_rank * Fe, Fe, Fe, j))
            s2.append(_cols(f"{m}experts.{e}.down_proj.weight", (H, Fm), etp_rank * Fe, Fe, 0, j))
        out.append(Leaf(pre + "w13", (El, 2 * Fe, H), "normal", s13))
        out.append(Leaf(pre + "w2", (El, H, Fe), "normal", s2))
        if arch.n_shared_experts:
            Fs = arch.n_shared_experts * Fm
            sh = mlp_leaves(pre + "shared_", m + "shared_experts.", Fs, True)
            out.extend(sh)
        if arch.shared_expert_intermediate_size:
            # Qwen3-Next: one shared expert whose output is scaled by sigmoid(x · gate)
            out.extend(mlp_leaves(pre + "shared_", m + "shared_expert.", arch.shared_expert_intermediate_size, True))
            out.append(_full(pre + "shared_expert_gate", (1, H), m + "shared_expert_gate.weight"))
    else:
        out.extend(mlp_leaves(pre, hp + "mlp.", arch.intermediate_size, True))
    for lf in out:
        if len(lf.segments) == 1 and lf.segments[0].extent == lf.segments[0].hf_shape:
            lf.replicated = True
    return out


def embed_leaves(arch: ModelArch, tp: int = 1, tp_rank: int = 0) -> List[Leaf]:
    V, H = arch.vocab_size, arch.hidden_size
    assert V % tp == 0
    Vl = V // tp
    return [Leaf("embed_tokens", (Vl, H), "normal",
                 [_rows("model.embed_tokens.weight", (V, H), tp_rank * Vl, Vl, 0)], tp == 1)]


def head_leaves(arch: ModelArch, tp: int = 1, tp_rank: int = 0) -> List[Leaf]:
    V, H = arch.vocab_size, arch.hidden_size
    out = [_full("norm", (H,), "model.norm.weight", "zeros" if arch.zero_centered_norm else "ones")]
    if arch.num_labels > 0:
        out.append(_full("score", (arch.num_labels, H), "score.weight"))
    elif not arch.tie_word_embeddings:
        Vl = V // tp
        out.append(Leaf("lm_head", (Vl, H), "normal",
                        [_rows("lm_head.weight", (V, H), tp_rank * Vl, Vl, 0)], tp == 1))
    return out


def model_blocks(arch: ModelArch, tp=1, tp_rank=0, ep=1, ep_rank=0,
                 layer_range: Optional[Tuple[int, int]] = None,
                 with_embed=True, with_head=True, etp=1, etp_rank=0) -> List[Tuple[str, List[Leaf]]]:
    """Blocks (= FSDP units / offload units) of a model instance in forward order.
    ``layer_range`` selects a pipeline stage's layers: one ``(lo, hi)`` pair, or a list of pairs when the
    stage holds several model chunks (interleaved pipeline schedule)."""
    ranges = layer_range or (0, arch.num_hidden_layers)
    if ranges and isinstance(ranges[0], int):
        ranges = [tuple(ranges)]
    blocks = []
    if with_embed:
        blocks.append(("embed", embed_leaves(arch, tp, tp_rank)))
    for lo, hi in ranges:
        for l in range(lo, hi):
            leaves = layer_leaves(arch, l, tp, tp_rank, ep, ep_rank, etp, etp_rank)
            experts = [lf for lf in leaves if lf.name.endswith((".w13", ".w2"))]
            blocks.append((f"layer{l}", [lf for lf in leaves if lf not in experts]))
            if experts:
                # expert weights are replicated over a different group (expert-DP), so
                # they shard, reduce and offload as a block of their own
                blocks.append((f"layer{l}.experts", experts))
    if with_head:
        blocks.append(("head", head_leaves(arch, tp, tp_rank)))
    return blocks


def hf_tensor_shapes(arch: ModelArch) -> Dict[str, Tuple[int, ...]]:
    """Name → shape of every tensor of the HF checkpoint of ``arch``."""
    shapes: Dict[str, Tuple[int, ...]] = {}
    for _, leaves in model_blocks(arch):
        for lf in leaves:
            for s in lf.segments:
                shapes[s.hf_name] = (s.hf_shape[0],) if len(lf.shape) == 1 else tuple(s.hf_shape)
                if s.hf_name.endswith(".conv1d.weight"):       # depthwise Conv1d: [channels, 1, taps]
                    shapes[s.hf_name] = (s.hf_shape[0], 1, s.hf_shape[1])
    return shapes
