"""Qwen3-Next (gated delta-net hybrid) against the HuggingFace implementation on CPU: logits of a
packed row, greedy generation through the rollout engine (chunked prefill, preemption), the
chunk-wise delta rule against the token-by-token recurrence, gradients."""
import pytest
import torch

from chatlearn_b200.models.nn import PRESETS, CausalLM
from chatlearn_b200.models.nn.hybrid import gated_delta_chunked, gated_delta_step
from chatlearn_b200.models.nn.model import packed_ctx

transformers = pytest.importorskip("transformers")


def _models():
    from transformers import Qwen3NextConfig, Qwen3NextForCausalLM
    torch.manual_seed(0)
    arch = PRESETS["tiny_qwen3_next"]()
    m = CausalLM(arch).init_weights(3, std=0.05)
    for _, p, lf, _ in m.named_leaves():
        if lf.init in ("zeros", "ones"):                      # norm scales away from their initial value
            p.add_(0.1 * torch.randn_like(p))
    cfg = Qwen3NextConfig(
        vocab_size=arch.vocab_size, hidden_size=arch.hidden_size, num_hidden_layers=arch.num_hidden_layers,
        num_attention_heads=arch.num_attention_heads, num_key_value_heads=arch.num_key_value_heads,
        head_dim=arch.head_dim, intermediate_size=arch.intermediate_size,
        moe_intermediate_size=arch.moe_intermediate_size, num_experts=arch.num_experts,
        num_experts_per_tok=arch.num_experts_per_tok,
        shared_expert_intermediate_size=arch.shared_expert_intermediate_size, norm_topk_prob=True,
        linear_num_key_heads=arch.linear_num_key_heads, linear_num_value_heads=arch.linear_num_value_heads,
        linear_key_head_dim=arch.linear_key_head_dim, linear_value_head_dim=arch.linear_value_head_dim,
        linear_conv_kernel_dim=arch.linear_conv_kernel_dim, rms_norm_eps=arch.rms_norm_eps,
        tie_word_embeddings=False, layer_types=arch.layer_types, decoder_sparse_step=1, mlp_only_layers=[],
        rope_parameters={"rope_type": "default", "rope_theta": arch.rope_theta, "partial_rotary_factor": 0.25},
        attn_implementation="eager")
    hf = Qwen3NextForCausalLM(cfg).eval()
    sd = m.hf_state_dict()
    conv = {k: v for k, v in sd.items() if ".mlp.experts." not in k}
    for l in range(arch.num_hidden_layers):                   # HF keeps the routed experts stacked
        pre = f"model.layers.{l}.mlp.experts."
        conv[pre + "gate_up_proj"] = torch.stack(
            [torch.cat([sd[f"{pre}{e}.gate_proj.weight"], sd[f"{pre}{e}.up_proj.weight"]], 0)
             for e in range(arch.num_experts)])
        conv[pre + "down_proj"] = torch.stack([sd[f"{pre}{e}.down_proj.weight"] for e in range(arch.num_experts)])
    missing, unexpected = hf.load_state_dict(conv, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    return arch, m, hf


def test_config_round_trip():
    arch = PRESETS["tiny_qwen3_next"]()
    assert arch.layer_types == ["linear_attention"] * 3 + ["full_attention"] and arch.rotary_dim == 8
    from chatlearn_b200.models.nn.arch import ModelArch
    again = ModelArch.from_hf_dict({
        "model_type": "qwen3_next", "vocab_size": 512, "hidden_size": 128, "num_hidden_layers": 8,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 32, "full_attention_interval": 4,
        "rope_parameters": {"rope_type": "default", "rope_theta": 5e6, "partial_rotary_factor": 0.25},
        "linear_num_key_heads": 2, "linear_num_value_heads": 4, "linear_key_head_dim": 16,
        "linear_value_head_dim": 16, "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 64,
        "shared_expert_intermediate_size": 64})
    assert again.layer_types[3] == again.layer_types[7] == "full_attention" and again.layer_is_linear(4)
    assert again.rope_theta == 5e6 and again.partial_rotary_factor == 0.25 and again.zero_centered_norm
    m = CausalLM(arch)
    assert m.num_params() == arch.num_params()
    shapes = {k: tuple(v.shape) for k, v in m.hf_state_dict().items()}
    assert shapes["model.layers.0.linear_attn.conv1d.weight"] == (2 * 32 + 64, 1, 4)
    assert shapes["model.layers.3.self_attn.q_proj.weight"] == (4 * 32 * 2, 128)
    assert shapes["model.layers.0.mlp.shared_expert_gate.weight"] == (1, 128)


def test_logits_match_hf_on_a_packed_row():
    arch, m, hf = _models()
    lens = [5, 70, 9, 64]
    toks = torch.randint(0, arch.vocab_size, (sum(lens),))
    ctx, _ = packed_ctx(lens, "cpu")
    with torch.no_grad():
        ours = m.logits(m.hidden_states(toks, ctx))
        o = 0
        for n in lens:
            ref = hf(toks[o:o + n][None]).logits[0]
            assert torch.allclose(ours[o:o + n], ref, atol=2e-4, rtol=1e-3), (n, float((ours[o:o + n] - ref).abs().max()))
            o += n


def test_engine_greedy_generation_matches_hf():
    from chatlearn_b200.rollout.engine import RolloutEngine, SamplingParams
    arch, m, hf = _models()
    prompts = [torch.randint(0, 500, (n,)).tolist() for n in (5, 23, 70, 9)]
    want = []
    for pr in prompts:
        with torch.no_grad():
            want.append(hf.generate(torch.tensor([pr]), max_new_tokens=12, do_sample=False, eos_token_id=None,
                                    pad_token_id=0)[0, len(pr):].tolist())
    preempted = 0
    # whole prompts; prompts fed in chunks of 16 tokens (state carried between chunks); a cache so small
    # that sequences are evicted and recomputed from an empty state
    for kw in (dict(), dict(max_num_batched_tokens=16), dict(num_blocks=7, block_size=16, max_num_seqs=3)):
        eng = RolloutEngine(m, max_model_len=256, **kw)
        outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
        assert [s.output for s in outs] == want, kw
        preempted += sum(s.preemptions for s in outs)
        assert not eng._state_slot                           # every finished sequence gave its slot back
    assert preempted > 0


def test_chunked_delta_rule_equals_recurrence_and_differentiates():
    torch.manual_seed(1)
    B, L, H, dk, dv = 2, 150, 3, 8, 6
    q = torch.nn.functional.normalize(torch.randn(B, L, H, dk), dim=-1) / dk ** 0.5
    k = torch.nn.functional.normalize(torch.randn(B, L, H, dk), dim=-1)
    v = torch.randn(B, L, H, dv)
    g = -torch.rand(B, L, H) * 0.5
    beta = torch.rand(B, L, H)
    S0 = torch.randn(B, H, dk, dv) * 0.1
    S, outs = S0, []
    for t in range(L):
        o, S = gated_delta_step(q[:, t], k[:, t], v[:, t], g[:, t], beta[:, t], S)
        outs.append(o)
    want = torch.stack(outs, 1)
    got, S_end = gated_delta_chunked(q, k, v, g, beta, S0)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-4)
    assert torch.allclose(S_end, S, atol=1e-5, rtol=1e-4)
    # neutral padding (no decay, no write) leaves outputs and the final state untouched
    pad = lambda t: torch.nn.functional.pad(t, (0, 0) * (t.dim() - 2) + (0, 37))      # noqa: E731
    kp, vp = pad(k), pad(v)
    kp[:, L:], vp[:, L:] = 1.0, 1.0                          # whatever the padded rows hold
    got_p, S_p = gated_delta_chunked(pad(q), kp, vp, pad(g), pad(beta), S0)
    assert torch.allclose(got_p[:, :L], want, atol=1e-5, rtol=1e-4) and torch.allclose(S_p, S, atol=1e-5, rtol=1e-4)
    # gradients flow through the triangular solve
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    gated_delta_chunked(qg, kg, vg, g, beta)[0].square().sum().backward()
    assert all(torch.isfinite(t.grad).all() and t.grad.abs().sum() > 0 for t in (qg, kg, vg))


def test_model_gradients_match_hf():
    arch, m, hf = _models()
    lens = [40, 70]
    toks = torch.randint(0, arch.vocab_size, (sum(lens),))
    labels = torch.randint(0, arch.vocab_size, (sum(lens),))
    for b in m.blocks:
        b.enable_grad(torch.zeros_like(b.flat))
    ctx, _ = packed_ctx(lens, "cpu")
    lp, _ = m.logprobs(toks, labels, ctx)
    (-lp.sum()).backward()
    hf.zero_grad()
    o, loss = 0, 0.0
    for n in lens:
        logits = hf(toks[o:o + n][None]).logits[0]
        loss = loss - torch.log_softmax(logits.float(), -1).gather(1, labels[o:o + n, None]).sum()
        o += n
    loss.backward()
    grads = {}
    for name, p, lf, b in m.named_leaves():
        grads[name] = p.grad
    hfp = dict(hf.named_parameters())
    g0 = grads["layers.0.in_proj"]
    ref = torch.cat([hfp["model.layers.0.linear_attn.in_proj_qkvz.weight"].grad,
                     hfp["model.layers.0.linear_attn.in_proj_ba.weight"].grad], 0)
    assert float((g0 - ref).norm() / ref.norm()) < 1e-3
    for ours_name, hf_name in (("layers.0.A_log", "model.layers.0.linear_attn.A_log"),
                               ("layers.1.conv1d", "model.layers.1.linear_attn.conv1d.weight"),
                               ("layers.3.q_norm", "model.layers.3.self_attn.q_norm.weight"),
                               ("layers.2.shared_expert_gate", "model.layers.2.mlp.shared_expert_gate.weight"),
                               ("layers.3.input_layernorm", "model.layers.3.input_layernorm.weight")):
        a, b_ = grads[ours_name], hfp[hf_name].grad.reshape(grads[ours_name].shape)
        assert float((a - b_).norm() / b_.norm()) < 1e-3, (ours_name, float((a - b_).abs().max()))


_TP_SCRIPT = r'''
import json, os, torch, torch.distributed as dist
from chatlearn_b200.models.nn import PRESETS, CausalLM
from chatlearn_b200.parallel.groups import Group
from chatlearn_b200.rollout.engine import RolloutEngine, SamplingParams
dist.init_process_group("gloo")
rank = dist.get_rank()
arch = PRESETS["tiny_qwen3_next"]()
full = CausalLM(arch, dtype=torch.float32).init_weights(5, std=0.05)
g = torch.Generator().manual_seed(3)
prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (5, 23, 70, 9)]
sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
want = [s.output for s in RolloutEngine(full, max_model_len=256).generate(prompts, sp)]
shard = CausalLM(arch, dtype=torch.float32, tp=2, tp_rank=rank)
shard.load_hf_state_dict(full.hf_state_dict())
tp = Group(dist.group.WORLD, [0, 1], "tp")
# whole prompts, then prompts in chunks of 16 tokens with the state carried between the chunks
got = [[s.output for s in RolloutEngine(shard, tp_group=tp, max_model_len=256, **kw).generate(prompts, sp)]
       for kw in (dict(), dict(max_num_batched_tokens=16))]
print("RESULT " + json.dumps({"rank": rank, "same": [g == want for g in got]}))
'''


def test_tensor_parallel_engine_generates_the_same_tokens():
    """Two tensor-parallel ranks, each with half of the heads of every mixer (and the recurrent state of those
    heads), generate token for token what one rank generates."""
    import json

    from tests.dist_utils import run_ranks
    outs, _ = run_ranks(_TP_SCRIPT, 2)
    res = [json.loads(line[7:]) for o in outs for line in o.splitlines() if line.startswith("RESULT ")]
    assert len(res) == 2 and all(r["same"] == [True, True] for r in res), res
