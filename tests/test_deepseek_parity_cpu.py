"""DeepSeek-V3 / Moonlight family (latent attention, sigmoid router with grouped top-k and a bias, shared
experts) against the HuggingFace implementation on CPU, with the rotary layout of the released
checkpoints and with the YaRN long-context rescaling."""
import pytest
import torch

from chatlearn_b200.models.nn import PRESETS, CausalLM
from chatlearn_b200.models.nn.arch import ModelArch
from chatlearn_b200.models.nn.model import packed_ctx

transformers = pytest.importorskip("transformers")

YARN = {"rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 16, "beta_fast": 32, "beta_slow": 1,
        "mscale": 1.0, "mscale_all_dim": 0.7}


@pytest.mark.parametrize("interleave,yarn,q_lora", [(True, False, None), (False, False, 24), (True, True, None)])
def test_logits_match_hf(interleave, yarn, q_lora):
    from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
    torch.manual_seed(0)
    arch = PRESETS["tiny_mla_moe"]()
    arch.rope_interleave, arch.q_lora_rank = interleave, q_lora
    arch.rope_scaling = dict(YARN) if yarn else None
    m = CausalLM(arch).init_weights(3, std=0.05)
    for _, p, lf, _ in m.named_leaves():
        if lf.init in ("zeros", "ones"):
            p.add_(0.1 * torch.randn_like(p))
    rp = {"rope_theta": arch.rope_theta, **(YARN if yarn else {"rope_type": "default"})}
    cfg = DeepseekV3Config(
        vocab_size=arch.vocab_size, hidden_size=arch.hidden_size, num_hidden_layers=arch.num_hidden_layers,
        num_attention_heads=arch.num_attention_heads, num_key_value_heads=arch.num_key_value_heads,
        intermediate_size=arch.intermediate_size, moe_intermediate_size=arch.moe_intermediate_size,
        n_routed_experts=arch.num_experts, num_experts_per_tok=arch.num_experts_per_tok,
        n_shared_experts=arch.n_shared_experts, first_k_dense_replace=arch.first_k_dense_replace,
        n_group=arch.n_group, topk_group=arch.topk_group, routed_scaling_factor=arch.routed_scaling_factor,
        norm_topk_prob=True, kv_lora_rank=arch.kv_lora_rank, q_lora_rank=q_lora,
        qk_nope_head_dim=arch.qk_nope_head_dim, qk_rope_head_dim=arch.qk_rope_head_dim, v_head_dim=arch.v_head_dim,
        rms_norm_eps=arch.rms_norm_eps, rope_parameters=rp, max_position_embeddings=128, tie_word_embeddings=False,
        attn_implementation="eager", rope_interleave=interleave)
    hf = DeepseekV3ForCausalLM(cfg).eval()
    sd = m.hf_state_dict()
    conv = {k: v for k, v in sd.items() if ".mlp.experts." not in k}
    for l in range(arch.first_k_dense_replace, arch.num_hidden_layers):       # HF keeps the routed experts stacked
        pre = f"model.layers.{l}.mlp.experts."
        conv[pre + "gate_up_proj"] = torch.stack(
            [torch.cat([sd[f"{pre}{e}.gate_proj.weight"], sd[f"{pre}{e}.up_proj.weight"]], 0)
             for e in range(arch.num_experts)])
        conv[pre + "down_proj"] = torch.stack([sd[f"{pre}{e}.down_proj.weight"] for e in range(arch.num_experts)])
    missing, unexpected = hf.load_state_dict(conv, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    lens = [7, 60]
    toks = torch.randint(0, arch.vocab_size, (sum(lens),))
    ctx, _ = packed_ctx(lens, "cpu")
    with torch.no_grad():
        ours = m.logits(m.hidden_states(toks, ctx))
        o = 0
        for n in lens:
            ref = hf(toks[o:o + n][None]).logits[0]
            assert torch.allclose(ours[o:o + n], ref, atol=2e-4, rtol=1e-3), (n, float((ours[o:o + n] - ref).abs().max()))
            o += n


def test_released_config_is_understood():
    arch = ModelArch.from_hf_dict({
        "model_type": "deepseek_v3", "vocab_size": 129280, "hidden_size": 7168, "num_hidden_layers": 61,
        "num_attention_heads": 128, "kv_lora_rank": 512, "q_lora_rank": 1536, "qk_nope_head_dim": 128,
        "qk_rope_head_dim": 64, "v_head_dim": 128, "n_routed_experts": 256, "num_experts_per_tok": 8,
        "moe_intermediate_size": 2048, "n_shared_experts": 1, "first_k_dense_replace": 3, "scoring_func": "sigmoid",
        "n_group": 8, "topk_group": 4, "routed_scaling_factor": 2.5, "rope_theta": 10000,
        "rope_scaling": {"type": "yarn", "factor": 40, "original_max_position_embeddings": 4096, "beta_fast": 32,
                         "beta_slow": 1, "mscale": 1.0, "mscale_all_dim": 1.0}})
    assert arch.use_mla and arch.rope_interleave and arch.rope_scaling["factor"] == 40 and arch.num_experts == 256
    from chatlearn_b200.models.nn.mla import attention_scale, yarn_inv_freq
    inv, att = yarn_inv_freq(64, 10000.0, arch.rope_scaling)
    assert att == 1.0 and inv.shape == (32,)
    assert abs(float(inv[0]) - 1.0) < 1e-6 and abs(float(inv[-1]) * 40 - 10000.0 ** (-62 / 64)) < 1e-7
    assert abs(attention_scale(arch) - (192 ** -0.5) * (0.1 * torch.log(torch.tensor(40.0)).item() + 1) ** 2) < 1e-6
