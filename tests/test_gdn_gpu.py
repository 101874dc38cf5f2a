"""Gated delta-net decode kernel against the PyTorch recurrence (fp32), and the Qwen3-Next
rollout path on the GPU against the same engine on PyTorch statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(q, k, v, g, beta, state, slots, fresh, scale):
    from chatlearn_b200.models.nn.hybrid import _l2norm, gated_delta_step
    r = v.shape[1] // q.shape[1]
    qn = (_l2norm(q.float()) * scale).repeat_interleave(r, dim=1)
    kn = _l2norm(k.float()).repeat_interleave(r, dim=1)
    S0 = state.index_select(0, slots) * (~fresh).float()[:, None, None, None]
    o, S = gated_delta_step(qn, kn, v.float(), g, beta, S0)
    state = state.clone()
    state.index_copy_(0, slots, S)
    return o, state


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(5, 2, 4, 16, 16), (64, 16, 32, 128, 128), (3, 4, 4, 64, 96)])
def test_gdn_decode_step_matches_recurrence(dtype, shape):
    from chatlearn_b200.ops import native
    B, nk, nv, dk, dv = shape
    dev = torch.device("cuda")
    torch.manual_seed(B)
    q = torch.randn(B, nk, dk, device=dev).to(dtype)
    k = torch.randn(B, nk, dk, device=dev).to(dtype)
    v = torch.randn(B, nv, dv, device=dev).to(dtype)
    g = -torch.rand(B, nv, device=dev)
    beta = torch.rand(B, nv, device=dev)
    state = torch.randn(B + 3, nv, dk, dv, device=dev) * 0.2
    slots = torch.randperm(B + 3, device=dev)[:B]
    fresh = torch.rand(B, device=dev) < 0.3
    want_o, want_S = _reference(q, k, v, g, beta, state, slots, fresh, dk ** -0.5)
    got_S = state.clone()
    got_o = native.C.gdn_decode_step(q, k, v, g, beta, got_S, slots, fresh, dk ** -0.5)
    torch.cuda.synchronize()
    assert torch.allclose(got_o, want_o, atol=2e-4, rtol=2e-4), float((got_o - want_o).abs().max())
    assert torch.allclose(got_S, want_S, atol=2e-4, rtol=2e-4), float((got_S - want_S).abs().max())


def test_qwen3_next_engine_native_matches_statements():
    from chatlearn_b200 import ops
    from chatlearn_b200.models.nn import PRESETS, CausalLM
    from chatlearn_b200.ops import native
    from chatlearn_b200.rollout.engine import RolloutEngine, SamplingParams
    arch = PRESETS["tiny_qwen3_next"]()
    m = CausalLM(arch, dtype=torch.float32, device="cuda").init_weights(5, std=0.05)
    prompts = [torch.randint(0, 500, (n,)).tolist() for n in (5, 23, 70, 9, 1)]
    outs = {}
    for mode in ("native", "library"):
        ops.set_mode(mode)
        try:
            eng = RolloutEngine(m, max_model_len=256, num_blocks=64, block_size=16, max_num_batched_tokens=48)
            before = native.launch_counts["gdn_decode_step"]
            seqs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
            outs[mode] = ([s.output for s in seqs], [s.logprobs for s in seqs])
            if mode == "native":
                assert native.launch_counts["gdn_decode_step"] > before
        finally:
            ops.set_mode("native")
    lp_n = torch.tensor(outs["native"][1])
    lp_r = torch.tensor(outs["library"][1])
    # fp32 weights: only the state update differs between the two runs (kernel against statements)
    assert [o[:4] for o in outs["native"][0]] == [o[:4] for o in outs["library"][0]]
    assert float((lp_n[:, :4] - lp_r[:, :4]).abs().max()) < 1e-3


def test_qwen3_next_decode_in_captured_steps():
    """bf16 weights: decode steps of the hybrid model are captured in CUDA graphs (state slots are graph inputs,
    padded rows update a scratch slot); tokens equal those of eager steps."""
    from chatlearn_b200.models.nn import PRESETS, CausalLM
    from chatlearn_b200.rollout.engine import RolloutEngine, SamplingParams
    arch = PRESETS["tiny_qwen3_next"]()
    m = CausalLM(arch, dtype=torch.bfloat16, device="cuda").init_weights(5, std=0.05)
    prompts = [torch.randint(0, 500, (n,)).tolist() for n in (5, 23, 70)]
    outs = {}
    for graphs in (True, False):
        eng = RolloutEngine(m, max_model_len=256, num_blocks=64, block_size=16, use_cuda_graphs=graphs)
        seqs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
        outs[graphs] = [s.output for s in seqs]
        assert bool(eng._graphs) == graphs
    assert outs[True] == outs[False]
