"""Text model families against their HuggingFace implementations on CPU (fp32): logits of a packed row
after loading this framework's HF-named state dict into the HF module."""
import pytest
import torch

from chatlearn_b200.models.nn import PRESETS, CausalLM
from chatlearn_b200.models.nn.model import packed_ctx

transformers = pytest.importorskip("transformers")


def _hf_model(arch):
    import transformers as tf
    common = dict(vocab_size=arch.vocab_size, hidden_size=arch.hidden_size, num_hidden_layers=arch.num_hidden_layers,
                  num_attention_heads=arch.num_attention_heads, num_key_value_heads=arch.num_key_value_heads,
                  intermediate_size=arch.intermediate_size, rms_norm_eps=arch.rms_norm_eps,
                  rope_parameters={"rope_type": "default", "rope_theta": arch.rope_theta},
                  max_position_embeddings=256, tie_word_embeddings=arch.tie_word_embeddings,
                  attn_implementation="eager")
    if arch.model_type == "llama":
        return tf.LlamaForCausalLM(tf.LlamaConfig(**common))
    if arch.model_type == "qwen2":
        return tf.Qwen2ForCausalLM(tf.Qwen2Config(**common))
    if arch.model_type == "qwen3":
        return tf.Qwen3ForCausalLM(tf.Qwen3Config(head_dim=arch.head_dim, **common))
    assert arch.model_type == "qwen3_moe"
    return tf.Qwen3MoeForCausalLM(tf.Qwen3MoeConfig(
        head_dim=arch.head_dim, moe_intermediate_size=arch.moe_intermediate_size, num_experts=arch.num_experts,
        num_experts_per_tok=arch.num_experts_per_tok, norm_topk_prob=arch.norm_topk_prob, decoder_sparse_step=1,
        mlp_only_layers=[], **common))


def _qwen2_tiny():
    a = PRESETS["tiny_llama"]()
    a.model_type, a.attention_bias, a.num_key_value_heads, a.rope_theta = "qwen2", True, 2, 1e6
    return a


def _tied():
    a = PRESETS["tiny_qwen3"]()
    a.tie_word_embeddings = True
    return a


@pytest.mark.parametrize("name,make", [("llama", PRESETS["tiny_llama"]), ("qwen2", _qwen2_tiny),
                                       ("qwen3", PRESETS["tiny_qwen3"]), ("qwen3_tied", _tied),
                                       ("qwen3_moe", PRESETS["tiny_moe"])])
def test_logits_match_hf(name, make):
    torch.manual_seed(0)
    arch = make()
    m = CausalLM(arch).init_weights(3, std=0.05)
    for _, p, lf, _ in m.named_leaves():
        if lf.init in ("zeros", "ones"):                      # biases and norm scales away from their initial value
            p.add_(0.1 * torch.randn_like(p))
    hf = _hf_model(arch).eval()
    sd = m.hf_state_dict()
    conv = {k: v for k, v in sd.items() if ".mlp.experts." not in k}
    if arch.is_moe:                                           # HF keeps the routed experts stacked
        for l in range(arch.num_hidden_layers):
            pre = f"model.layers.{l}.mlp.experts."
            conv[pre + "gate_up_proj"] = torch.stack(
                [torch.cat([sd[f"{pre}{e}.gate_proj.weight"], sd[f"{pre}{e}.up_proj.weight"]], 0)
                 for e in range(arch.num_experts)])
            conv[pre + "down_proj"] = torch.stack([sd[f"{pre}{e}.down_proj.weight"] for e in range(arch.num_experts)])
    missing, unexpected = hf.load_state_dict(conv, strict=False)
    assert not unexpected and all(k == "lm_head.weight" and arch.tie_word_embeddings for k in missing), (missing, unexpected)
    lens = [9, 40]
    toks = torch.randint(0, arch.vocab_size, (sum(lens),))
    ctx, _ = packed_ctx(lens, "cpu")
    with torch.no_grad():
        ours = m.logits(m.hidden_states(toks, ctx))
        o = 0
        for n in lens:
            ref = hf(toks[o:o + n][None]).logits[0]
            assert torch.allclose(ours[o:o + n], ref, atol=2e-4, rtol=1e-3), (n, float((ours[o:o + n] - ref).abs().max()))
            o += n
