"""Model architecture description (HuggingFace ``config.json`` compatible).

One dataclass covers the families the reference trains: Llama-2, Qwen2.5/Qwen3
dense, Qwen3-MoE, and DeepSeek-V3 / Moonlight (MLA attention + sigmoid-routed
MoE with shared experts).  The reference reads these through ``AutoConfig`` and
converts them for Megatron in chatlearn/utils/megatron_utils.py:20-164; here the
same HF keys are read directly.
"""
import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class ModelArch:
    model_type: str = "qwen3"            # llama | qwen2 | qwen3 | qwen3_moe | deepseek_v3
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    intermediate_size: int = 11008
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 32768
    qk_norm: bool = False                # Qwen3 per-head RMSNorm on q and k
    attention_bias: bool = False         # Qwen2 qkv bias
    tie_word_embeddings: bool = False
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    n_shared_experts: int = 0
    first_k_dense_replace: int = 0       # leading dense layers (DeepSeek/Moonlight)
    scoring_func: str = "softmax"        # softmax | sigmoid
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    router_bias: bool = False            # e_score_correction_bias (aux-free balancing)
    # MLA
    use_mla: bool = False
    kv_lora_rank: int = 0
    q_lora_rank: Optional[int] = None
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    rope_interleave: Optional[bool] = None   # rotary dims stored as (even, odd) pairs (DeepSeek checkpoints); None: by family
    rope_scaling: Optional[Dict[str, Any]] = None   # {"type": "yarn", "factor", "original_max_position_embeddings", ...}
    # vision-language models: rotary sections (time, row, column) and the vision tower's config
    mrope_section: Optional[List[int]] = None
    mrope_interleaved: bool = False      # Qwen3-VL frequency layout
    vision_config: Optional[Dict[str, Any]] = None
    image_token_id: Optional[int] = None
    video_token_id: Optional[int] = None             # placeholder of video frames (same tower, own temporal positions)
    # Qwen3-Next: gated delta-net ("linear_attention") layers interleaved with gated full attention
    layer_types: Optional[List[str]] = None          # per layer: "linear_attention" | "full_attention"
    full_attention_interval: int = 4                 # default pattern when layer_types is not given
    partial_rotary_factor: float = 1.0               # fraction of the head dim that rotates
    attn_output_gate: bool = False                   # q_proj also emits a per-channel sigmoid gate
    zero_centered_norm: bool = False                 # RMSNorm scales by (1 + weight)
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    shared_expert_intermediate_size: int = 0         # sigmoid-gated shared expert beside the routed ones
    # reward-model head
    num_labels: int = 0                  # >0: scalar/value head instead of lm_head
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    extra: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.model_type == "qwen3" or self.model_type == "qwen3_moe":
            self.qk_norm = True
        if self.model_type == "qwen2":
            self.attention_bias = True
        if self.model_type in ("deepseek_v3", "deepseek_v2", "kimi_k2", "moonlight"):
            self.use_mla = self.kv_lora_rank > 0
            if self.rope_interleave is None:
                self.rope_interleave = True      # the released checkpoints of this family pair up the rotary dims
        self.rope_interleave = bool(self.rope_interleave)
        if isinstance(self.rope_scaling, dict):
            kind = self.rope_scaling.get("rope_type", self.rope_scaling.get("type"))
            if kind != "yarn" or not self.use_mla:
                self.rope_scaling = None         # only the long-context rescaling of MLA models is modelled
        if self.model_type != "qwen3_next":
            self.layer_types = None          # other families list "full_attention" / sliding-window kinds there
        if self.model_type == "qwen3_next":
            self.qk_norm = self.attn_output_gate = self.zero_centered_norm = True
            if self.layer_types is None:
                k = max(int(self.full_attention_interval), 1)
                self.layer_types = ["full_attention" if (i + 1) % k == 0 else "linear_attention"
                                    for i in range(self.num_hidden_layers)]
        if self.eos_token_id is None:
            self.eos_token_id = self.vocab_size - 1

    # ---- derived sizes ----
    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def layer_is_moe(self, layer: int) -> bool:
        return self.is_moe and layer >= self.first_k_dense_replace

    def layer_is_linear(self, layer: int) -> bool:
        """Gated delta-net token mixer (recurrent state) instead of softmax attention."""
        return self.layer_types is not None and self.layer_types[layer] == "linear_attention"

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def q_size(self) -> int:
        if self.use_mla:
            return self.num_attention_heads * (self.qk_nope_head_dim + self.qk_rope_head_dim)
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def num_params(self) -> int:
        h, v = self.hidden_size, self.vocab_size
        n = v * h * (1 if self.tie_word_embeddings else 2) + h
        for l in range(self.num_hidden_layers):
            n += 2 * h
            if self.layer_is_linear(l):
                kd = self.linear_num_key_heads * self.linear_key_head_dim
                vd = self.linear_num_value_heads * self.linear_value_head_dim
                n += h * (2 * kd + 2 * vd + 2 * self.linear_num_value_heads) + vd * h
                n += (2 * kd + vd) * self.linear_conv_kernel_dim + 2 * self.linear_num_value_heads
                n += self.linear_value_head_dim
            elif self.use_mla:
                qd = self.qk_nope_head_dim + self.qk_rope_head_dim
                nh = self.num_attention_heads
                if self.q_lora_rank:
                    n += h * self.q_lora_rank + self.q_lora_rank + self.q_lora_rank * nh * qd
                else:
                    n += h * nh * qd
                n += h * (self.kv_lora_rank + self.qk_rope_head_dim) + self.kv_lora_rank
                n += self.kv_lora_rank * nh * (self.qk_nope_head_dim + self.v_head_dim)
                n += nh * self.v_head_dim * h
            else:
                n += h * (self.q_size * (2 if self.attn_output_gate else 1) + 2 * self.kv_size) + self.q_size * h
                if self.qk_norm:
                    n += 2 * self.head_dim
                if self.attention_bias:
                    n += self.q_size + 2 * self.kv_size
            if self.layer_is_moe(l):
                n += self.num_experts * h + (self.num_experts if self.router_bias else 0)
                n += self.num_experts * 3 * h * self.moe_intermediate_size
                n += self.n_shared_experts * 3 * h * self.moe_intermediate_size
                if self.shared_expert_intermediate_size:
                    n += 3 * h * self.shared_expert_intermediate_size + h
            else:
                n += 3 * h * self.intermediate_size
        return n

    # ---- HF config.json round trip ----
    _HF_ALIASES = {"num_local_experts": "num_experts", "n_routed_experts": "num_experts",
                   "norm_eps": "rms_norm_eps"}

    @classmethod
    def from_hf_dict(cls, d: Dict[str, Any]) -> "ModelArch":
        known = {f for f in cls.__dataclass_fields__}  # pylint: disable=no-member
        kw, extra = {}, {}
        if isinstance(d.get("text_config"), dict):
            # vision-language checkpoints nest the language model's settings
            outer = {k: v for k, v in d.items() if k != "text_config"}
            d = {**outer, **d["text_config"]}
            if "tie_word_embeddings" in outer:
                # the wrapping model decides whether the output head shares the embedding matrix
                d["tie_word_embeddings"] = outer["tie_word_embeddings"]
            d["model_type"] = {"qwen2_5_vl": "qwen2", "qwen2_5_vl_text": "qwen2", "qwen2_vl": "qwen2",
                               "qwen3_vl": "qwen3", "qwen3_vl_text": "qwen3", "qwen3_vl_moe": "qwen3_moe",
                               "qwen3_vl_moe_text": "qwen3_moe"}.get(d.get("model_type"), d.get("model_type"))
        rs = d.get("rope_scaling") or d.get("rope_parameters") or {}
        if isinstance(rs, dict) and rs.get("mrope_section"):
            d = dict(d, mrope_section=list(rs["mrope_section"]), mrope_interleaved=bool(rs.get("mrope_interleaved", False)))
            if "rope_theta" in rs and "rope_theta" not in d:
                d["rope_theta"] = rs["rope_theta"]
        if isinstance(rs, dict):
            # newer config files keep the rotary settings in one nested dict
            for key in ("rope_theta", "partial_rotary_factor"):
                if key in rs and key not in d:
                    d = dict(d, **{key: rs[key]})
            if rs.get("rope_type", rs.get("type")) == "yarn" and not d.get("rope_scaling"):
                d = dict(d, rope_scaling=dict(rs))
        for k, v in d.items():
            k = cls._HF_ALIASES.get(k, k)
            if k in known and k != "extra":
                kw[k] = v
            else:
                extra[k] = v
        arch = cls(**kw)
        arch.extra = extra
        return arch

    @property
    def visual_token_ids(self) -> Tuple[int, ...]:
        """Placeholder tokens whose rows take the vision tower's output."""
        return tuple(t for t in (self.image_token_id, self.video_token_id) if t is not None)

    @property
    def tokens_per_second(self) -> float:
        """Temporal positions per second of video (Qwen2.5-VL; 1 where the tower's settings do not say)."""
        return float((self.vision_config or {}).get("tokens_per_second", 1))

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelArch":
        with open(os.path.join(path, "config.json"), "r", encoding="utf-8") as f:
            return cls.from_hf_dict(json.load(f))

    def to_hf_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        extra = d.pop("extra")
        d.update(extra)
        arch_names = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM",
                      "qwen3": "Qwen3ForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM",
                      "deepseek_v3": "DeepseekV3ForCausalLM", "qwen3_next": "Qwen3NextForCausalLM"}
        d.setdefault("architectures", [arch_names.get(self.model_type, "LlamaForCausalLM")])
        if self.model_type == "deepseek_v3":
            d["n_routed_experts"] = self.num_experts
        return d

    def save_pretrained(self, path: str):
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as f:
            json.dump(self.to_hf_dict(), f, indent=2)


def resolve_arch(model_cfg) -> ModelArch:
    """Architecture of a role: inline ``model_arch`` dict, a preset name, or the
    ``config.json`` under ``load``."""
    ma = getattr(model_cfg, "model_arch", None)
    if isinstance(ma, ModelArch):
        return ma
    if isinstance(ma, str):
        return PRESETS[ma]()
    if isinstance(ma, dict) and ma:
        if "preset" in ma:
            arch = PRESETS[ma["preset"]]()
            for k, v in ma.items():
                if k != "preset":
                    setattr(arch, k, v)
            return arch
        return ModelArch.from_hf_dict(ma)
    load = getattr(model_cfg, "load", None)
    if load and os.path.exists(os.path.join(load, "config.json")):
        return ModelArch.from_pretrained(load)
    raise ValueError("model needs `model_arch` (inline dict / preset) or `load` with a config.json")


# ---- presets: the shapes named by the benchmark configurations ----

def tiny_qwen3() -> ModelArch:
    return ModelArch(model_type="qwen3", vocab_size=1024, hidden_size=256, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                     intermediate_size=704, rope_theta=1e6, rms_norm_eps=1e-6)


def qwen3_8b() -> ModelArch:
    return ModelArch(model_type="qwen3", vocab_size=151936, hidden_size=4096, num_hidden_layers=36,
                     num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                     intermediate_size=12288, rope_theta=1e6, rms_norm_eps=1e-6,
                     max_position_embeddings=40960)


def qwen3_30b_a3b() -> ModelArch:
    return ModelArch(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048,
                     num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4,
                     head_dim=128, intermediate_size=6144, moe_intermediate_size=768,
                     num_experts=128, num_experts_per_tok=8, norm_topk_prob=True,
                     router_aux_loss_coef=1e-3, rope_theta=1e6)


def llama2_7b() -> ModelArch:
    return ModelArch(model_type="llama", vocab_size=32000, hidden_size=4096, num_hidden_layers=32,
                     num_attention_heads=32, num_key_value_heads=32, intermediate_size=11008,
                     rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=4096)


def moonlight_16b_a3b() -> ModelArch:
    return ModelArch(model_type="deepseek_v3", vocab_size=163840, hidden_size=2048,
                     num_hidden_layers=27, num_attention_heads=16, num_key_value_heads=16,
                     intermediate_size=11264, moe_intermediate_size=1408, num_experts=64,
                     num_experts_per_tok=6, n_shared_experts=2, first_k_dense_replace=1,
                     scoring_func="sigmoid", n_group=1, topk_group=1, routed_scaling_factor=2.446,
                     norm_topk_prob=True, router_bias=True, kv_lora_rank=512, q_lora_rank=None,
                     qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, head_dim=192,
                     rope_theta=50000.0, rms_norm_eps=1e-5)


def tiny_moe() -> ModelArch:
    return ModelArch(model_type="qwen3_moe", vocab_size=512, hidden_size=128, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                     intermediate_size=256, moe_intermediate_size=64, num_experts=8,
                     num_experts_per_tok=2, router_aux_loss_coef=1e-3, rope_theta=1e6)


def tiny_mla_moe() -> ModelArch:
    return ModelArch(model_type="deepseek_v3", vocab_size=512, hidden_size=128, num_hidden_layers=3,
                     num_attention_heads=4, num_key_value_heads=4, intermediate_size=256,
                     moe_intermediate_size=64, num_experts=8, num_experts_per_tok=2,
                     n_shared_experts=1, first_k_dense_replace=1, scoring_func="sigmoid",
                     n_group=2, topk_group=1, routed_scaling_factor=1.5, router_bias=True,
                     kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                     head_dim=24, rope_theta=10000.0)


def tiny_llama() -> ModelArch:
    return ModelArch(model_type="llama", vocab_size=512, hidden_size=128, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=4, intermediate_size=352,
                     rope_theta=10000.0, rms_norm_eps=1e-5)


def tiny_qwen2_5_vl() -> ModelArch:
    """Qwen2.5-VL shape in miniature: Qwen2 language model with mrope + a windowed-attention vision tower."""
    return ModelArch(model_type="qwen2", vocab_size=1024, hidden_size=128, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, intermediate_size=256, rope_theta=1e6,
                     mrope_section=[4, 6, 6], image_token_id=1000, video_token_id=1001,
                     vision_config=dict(depth=2, hidden_size=64, intermediate_size=96, num_heads=4, patch_size=14,
                                        spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=128,
                                        window_size=56, fullatt_block_indexes=[1]))


def tiny_qwen3_vl() -> ModelArch:
    """Qwen3-VL shape in miniature: Qwen3 language model with the interleaved mrope layout + a vision tower with a
    learned position table whose early layers feed deep-stack taps into the first language layers."""
    return ModelArch(model_type="qwen3", vocab_size=1024, hidden_size=128, num_hidden_layers=3,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=32, intermediate_size=256, rope_theta=1e6,
                     mrope_section=[4, 6, 6], mrope_interleaved=True, image_token_id=1000, video_token_id=1001,
                     vision_config=dict(depth=3, hidden_size=64, intermediate_size=96, num_heads=4, patch_size=16,
                                        spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=128,
                                        num_position_embeddings=64, deepstack_visual_indexes=[0, 2]))


def qwen2_5_vl_7b() -> ModelArch:
    return ModelArch(model_type="qwen2", vocab_size=152064, hidden_size=3584, num_hidden_layers=28,
                     num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944, rope_theta=1e6,
                     mrope_section=[16, 24, 24], image_token_id=151655, video_token_id=151656,
                     vision_config=dict(depth=32, hidden_size=1280, intermediate_size=3420, num_heads=16, patch_size=14,
                                        spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=3584,
                                        window_size=112, fullatt_block_indexes=[7, 15, 23, 31]))


def qwen3_235b_a22b() -> ModelArch:
    return ModelArch(model_type="qwen3_moe", vocab_size=151936, hidden_size=4096, num_hidden_layers=94,
                     num_attention_heads=64, num_key_value_heads=4, head_dim=128, intermediate_size=12288,
                     moe_intermediate_size=1536, num_experts=128, num_experts_per_tok=8, norm_topk_prob=True,
                     router_aux_loss_coef=1e-3, rope_theta=1e6, max_position_embeddings=40960)


def deepseek_v3_671b() -> ModelArch:
    """DeepSeek-V3 shapes (the long-context rotary rescaling of the released checkpoint is not modelled)."""
    return ModelArch(model_type="deepseek_v3", vocab_size=129280, hidden_size=7168, num_hidden_layers=61,
                     num_attention_heads=128, num_key_value_heads=128, intermediate_size=18432,
                     moe_intermediate_size=2048, num_experts=256, num_experts_per_tok=8, n_shared_experts=1,
                     first_k_dense_replace=3, scoring_func="sigmoid", n_group=8, topk_group=4,
                     routed_scaling_factor=2.5, norm_topk_prob=True, router_bias=True, kv_lora_rank=512,
                     q_lora_rank=1536, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, head_dim=192,
                     rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=163840)


def tiny_qwen3_next() -> ModelArch:
    """Qwen3-Next in miniature: three gated delta-net layers per gated-attention layer, MoE with a
    sigmoid-gated shared expert, a quarter of each head rotating."""
    return ModelArch(model_type="qwen3_next", vocab_size=512, hidden_size=128, num_hidden_layers=4,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=32, partial_rotary_factor=0.25,
                     intermediate_size=256, moe_intermediate_size=64, num_experts=8, num_experts_per_tok=2,
                     shared_expert_intermediate_size=64, norm_topk_prob=True, rope_theta=1e6,
                     linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
                     linear_value_head_dim=16, linear_conv_kernel_dim=4)


def qwen3_next_80b_a3b() -> ModelArch:
    return ModelArch(model_type="qwen3_next", vocab_size=151936, hidden_size=2048, num_hidden_layers=48,
                     num_attention_heads=16, num_key_value_heads=2, head_dim=256, partial_rotary_factor=0.25,
                     intermediate_size=5120, moe_intermediate_size=512, num_experts=512, num_experts_per_tok=10,
                     shared_expert_intermediate_size=512, norm_topk_prob=True, router_aux_loss_coef=1e-3,
                     rope_theta=1e7, max_position_embeddings=262144,
                     linear_num_key_heads=16, linear_num_value_heads=32, linear_key_head_dim=128,
                     linear_value_head_dim=128, linear_conv_kernel_dim=4)


PRESETS = {
    "tiny_qwen3_next": tiny_qwen3_next, "qwen3_next_80b_a3b": qwen3_next_80b_a3b,
    "qwen3_235b_a22b": qwen3_235b_a22b, "deepseek_v3_671b": deepseek_v3_671b,
    "tiny_qwen2_5_vl": tiny_qwen2_5_vl, "tiny_qwen3_vl": tiny_qwen3_vl, "qwen2_5_vl_7b": qwen2_5_vl_7b,
    "tiny_qwen3": tiny_qwen3, "qwen3_8b": qwen3_8b, "qwen3_30b_a3b": qwen3_30b_a3b,
    "llama2_7b": llama2_7b, "moonlight_16b_a3b": moonlight_16b_a3b, "tiny_moe": tiny_moe,
    "tiny_mla_moe": tiny_mla_moe, "tiny_llama": tiny_llama,
}
