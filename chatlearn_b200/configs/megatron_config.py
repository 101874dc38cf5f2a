"""Megatron-style (TP/PP/CP/EP/ETP) trainer configuration.

Parity: chatlearn/configs/megatron_config.py:14-461.  Field names follow the
reference so its YAML templates load; the model described by
``MegatronModelArchitectureConfig`` is built by this framework's own
tensor/expert-parallel layers (chatlearn_b200/parallel), not by Megatron-Core.
"""
import math
from dataclasses import dataclass, field
from typing import Any, List, Optional

from .base import BaseConfig, BaseModelConfig
from .common import PolicyTrainerConfig, RefPolicyConfig
from .conf import MISSING


@dataclass
class MegatronModelArchitectureConfig(BaseConfig):
    attention_dropout: float = 0.0
    hidden_dropout: float = 0.0
    num_layers: int = MISSING
    hidden_size: int = MISSING
    num_attention_heads: int = MISSING
    ffn_hidden_size: int = MISSING
    num_query_groups: Optional[int] = None
    max_position_embeddings: int = MISSING
    swiglu: bool = True
    normalization: str = "RMSNorm"
    norm_epsilon: float = 1e-6
    position_embedding_type: str = "rope"
    mrope_section: Optional[Any] = None
    add_qkv_bias: bool = False
    add_bias_linear: bool = False
    rotary_base: int = 1000000
    rotary_percent: float = 1.0
    group_query_attention: bool = False
    untie_embeddings_and_output_weights: bool = False
    qk_layernorm: bool = False
    vocab_size: int = 32000
    kv_channels: int = MISSING
    # MoE
    num_experts: Optional[int] = None
    moe_grouped_gemm: bool = False
    moe_token_dispatcher_type: str = "allgather"
    moe_router_topk: int = 2
    moe_router_load_balancing_type: str = "none"
    moe_router_dtype: Optional[str] = None
    moe_router_pre_softmax: bool = False
    moe_permute_fusion: bool = False
    moe_router_fusion: bool = False
    moe_layer_freq: Any = 1
    moe_ffn_hidden_size: Optional[int] = None
    moe_aux_loss_coeff: float = 0.0
    moe_router_num_groups: Optional[int] = None
    moe_router_group_topk: Optional[int] = None
    moe_shared_expert_intermediate_size: Optional[int] = None
    moe_router_score_function: str = "softmax"
    moe_router_enable_expert_bias: bool = False
    moe_router_bias_update_rate: float = 1e-3
    moe_router_topk_scaling_factor: float = 0.0
    moe_shared_expert_overlap: bool = False
    # MLA
    multi_latent_attention: bool = False
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 32
    qk_head_dim: int = 128
    qk_pos_emb_head_dim: int = 64
    v_head_dim: Optional[int] = None
    # fusions (accepted; the native kernels are always fused)
    apply_rope_fusion: bool = True
    bias_swiglu_fusion: bool = True
    bias_dropout_fusion: bool = True
    rotary_scaling_factor: float = 1.0
    attention_backend: str = "auto"
    rope_type: Optional[str] = None
    cross_entropy_fusion_impl: str = "native"
    cross_entropy_loss_fusion: bool = False
    create_attention_mask_in_dataloader: bool = True
    async_tensor_model_parallel_allreduce: bool = False
    overlap_p2p_comm: bool = True
    batch_p2p_comm: bool = False
    deallocate_pipeline_outputs: bool = False
    overlap_moe_expert_parallel_comm: bool = False
    enable_experimental: bool = False
    freeze_LM: bool = False
    freeze_ViT: bool = False
    freeze_VP: bool = False
    hybrid_override_pattern: Optional[str] = None
    is_hybrid_model: bool = False
    apply_layernorm_1p: bool = False

    def _validate_impl(self):
        if self.num_experts is not None:
            assert self.moe_router_topk <= self.num_experts
            assert self.moe_router_score_function in ("softmax", "sigmoid")


@dataclass
class MegatronConfig(BaseConfig):
    model_provider_module: str = "pretrain_gpt"
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    context_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: Optional[int] = None
    virtual_pipeline_model_parallel_size: Optional[int] = None
    pipeline_model_parallel_layout: Optional[str] = None
    sequence_parallel: bool = True
    seq_length: int = MISSING
    tokenizer_type: str = "NullTokenizer"
    tokenizer_model: Optional[str] = None
    megatron_model_cfg: MegatronModelArchitectureConfig = field(
        default_factory=MegatronModelArchitectureConfig)
    decoder_first_pipeline_num_layers: Optional[int] = None
    decoder_last_pipeline_num_layers: Optional[int] = None
    moe_router_force_load_balancing: bool = False
    bf16: bool = True
    variable_seq_lengths: bool = False
    rerun_mode: str = "disabled"
    use_expandable_segments: bool = False

    def _post_init_impl(self):
        if isinstance(self, BaseModelConfig) and self.num_gpu:
            tp, cp = self.tensor_model_parallel_size, self.context_parallel_size
            pp, ep = self.pipeline_model_parallel_size, self.expert_model_parallel_size
            etp = self.expert_tensor_parallel_size or 1
            self.num_replica = 1
            if not self.trainable:
                self.num_replica = max(1, self.num_gpu // (math.lcm(tp * cp, etp * ep) * pp))
            self.replica_dp_size = max(1, self.num_gpu // (self.num_replica * tp * cp * pp))
            self.variable_seq_lengths = self.packing
            if self.variable_seq_lengths and self.megatron_model_cfg.num_experts is not None:
                # packed (variable-length) batches cannot use the all-gather dispatcher
                self.megatron_model_cfg.moe_token_dispatcher_type = "alltoall"
            self.seq_length = self.max_response_tokens_length + self.max_prompt_tokens_length

    def _validate_impl(self):
        if isinstance(self, BaseModelConfig):
            assert self.num_gpu > 0, "the Megatron-style backend needs at least one GPU"
            assert self.num_gpu % self.num_replica == 0
            tp, cp = self.tensor_model_parallel_size, self.context_parallel_size
            pp, ep = self.pipeline_model_parallel_size, self.expert_model_parallel_size
            etp = self.expert_tensor_parallel_size or 1
            assert self.num_gpu % (tp * cp * pp) == 0, "num_gpu must be a multiple of tp*cp*pp"
            assert self.num_gpu % (etp * ep * pp) == 0, "num_gpu must be a multiple of etp*ep*pp"
            if self.variable_seq_lengths:
                assert self.megatron_model_cfg.moe_token_dispatcher_type != "allgather" \
                    or self.megatron_model_cfg.num_experts is None, \
                    "packing needs the alltoall token dispatcher"


@dataclass
class MegatronRefPolicyConfig(RefPolicyConfig, MegatronConfig):
    pass


@dataclass
class MegatronPolicyTrainerConfig(PolicyTrainerConfig, MegatronConfig):
    recompute_granularity: Optional[str] = None
    recompute_method: Optional[str] = None
    recompute_num_layers: Optional[int] = None
    recompute_modules: Optional[List[str]] = None
    use_distributed_optimizer: bool = False
    no_load_optim: bool = True
    calculate_per_token_loss: bool = True
    gradient_accumulation_fusion: bool = False
    empty_unused_memory_level: Optional[int] = 0
    use_checkpoint_opt_param_scheduler: bool = True
    no_load_rng: bool = True
    no_load_scheduler: bool = True
    finetune: bool = True
    distributed_timeout_minutes: int = 10

    def _validate_impl(self):
        assert self.calculate_per_token_loss, "the GRPO loss is a per-token sum; keep calculate_per_token_loss=true"
        if self.recompute_granularity is not None:
            assert self.recompute_granularity in ("selective", "full")
