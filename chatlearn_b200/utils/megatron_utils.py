"""HF ``config.json`` → Megatron architecture config.

Parity: chatlearn/utils/megatron_utils.py:20-164 (``update_cfg``): for every
Megatron-backend role the architecture block ``megatron_model_cfg`` is filled from
the HuggingFace config of ``load`` (or the inline ``model_arch``): Qwen2.5/Qwen3
dense, Qwen2.5-VL (multimodal rotary sections), Qwen3-MoE, DeepSeek-V3 / Moonlight (MLA, sigmoid router,
group top-k, shared experts, YaRN factor), Qwen3-Next (hybrid layer pattern, partial rotary).  The parallel layers themselves read ``ModelArch``; this keeps
the reference's config surface populated for users and tools that inspect it.
"""
from chatlearn_b200.models.nn.arch import ModelArch, resolve_arch


def arch_to_megatron_cfg(arch: ModelArch, mc):
    mc.num_layers = arch.num_hidden_layers
    mc.hidden_size = arch.hidden_size
    mc.num_attention_heads = arch.num_attention_heads
    mc.ffn_hidden_size = arch.intermediate_size
    mc.num_query_groups = arch.num_key_value_heads
    mc.group_query_attention = arch.num_key_value_heads != arch.num_attention_heads
    mc.max_position_embeddings = arch.max_position_embeddings
    mc.norm_epsilon = arch.rms_norm_eps
    mc.rotary_base = int(arch.rope_theta)
    mc.vocab_size = arch.vocab_size
    mc.kv_channels = arch.head_dim
    mc.qk_layernorm = arch.qk_norm
    mc.add_qkv_bias = arch.attention_bias
    mc.untie_embeddings_and_output_weights = not arch.tie_word_embeddings
    mc.swiglu, mc.normalization, mc.position_embedding_type = True, "RMSNorm", "rope"
    if arch.is_moe:
        mc.num_experts = arch.num_experts
        mc.moe_router_topk = arch.num_experts_per_tok
        mc.moe_ffn_hidden_size = arch.moe_intermediate_size
        mc.moe_aux_loss_coeff = arch.router_aux_loss_coef
        mc.moe_router_load_balancing_type = "aux_loss" if arch.router_aux_loss_coef > 0 else "none"
        mc.moe_grouped_gemm = True
        mc.moe_token_dispatcher_type = "alltoall"
        mc.moe_router_dtype = "fp32"
        mc.moe_router_score_function = arch.scoring_func
        mc.moe_router_enable_expert_bias = arch.router_bias
        mc.moe_router_topk_scaling_factor = arch.routed_scaling_factor
        mc.moe_layer_freq = [0] * arch.first_k_dense_replace + \
            [1] * (arch.num_hidden_layers - arch.first_k_dense_replace)
        if arch.n_group > 1:
            mc.moe_router_num_groups, mc.moe_router_group_topk = arch.n_group, arch.topk_group
        if arch.n_shared_experts:
            mc.moe_shared_expert_intermediate_size = arch.n_shared_experts * arch.moe_intermediate_size
    if arch.use_mla:
        mc.multi_latent_attention = True
        mc.kv_lora_rank, mc.q_lora_rank = arch.kv_lora_rank, arch.q_lora_rank
        mc.qk_head_dim, mc.qk_pos_emb_head_dim = arch.qk_nope_head_dim, arch.qk_rope_head_dim
        mc.v_head_dim = arch.v_head_dim
        mc.kv_channels = arch.qk_nope_head_dim + arch.qk_rope_head_dim
        if arch.rope_scaling:                        # YaRN long-context rescaling (DeepSeek-V3)
            mc.rotary_scaling_factor = float(arch.rope_scaling.get("factor", 1.0))
    if arch.mrope_section:                           # vision-language models: time / row / column rotary sections
        mc.mrope_section = list(arch.mrope_section)
        mc.position_embedding_type = "mrope"
    if arch.layer_types is not None:                 # Qwen3-Next: "M-" = gated delta-net + MLP, "*-" = attention + MLP
        mc.hybrid_override_pattern = "".join("M-" if arch.layer_is_linear(l) else "*-"
                                             for l in range(arch.num_hidden_layers))
        mc.is_hybrid_model = True
        mc.rotary_percent = float(arch.partial_rotary_factor)
        if arch.shared_expert_intermediate_size:
            mc.moe_shared_expert_intermediate_size = arch.shared_expert_intermediate_size
    return mc


def update_cfg(cfg):
    for name in ("policy_trainer", "ref_policy"):
        m = getattr(cfg.models, name, None)
        if m is None or not hasattr(m, "megatron_model_cfg"):
            continue
        try:
            arch = resolve_arch(m)
        except ValueError:
            continue                      # architecture given explicitly in megatron_model_cfg
        arch_to_megatron_cfg(arch, m.megatron_model_cfg)
    return cfg
