"""Multi-head latent attention in the rollout engine: the cache holds one compressed row per token
(latent + rotary key) and decode attends in the latent space; the tokens must be the ones a full
recomputation of every prefix picks."""
import pytest
import torch

from chatlearn_b200.models.nn import PRESETS, CausalLM
from chatlearn_b200.models.nn.model import packed_ctx
from chatlearn_b200.rollout.engine import RolloutEngine, SamplingParams


def _greedy_by_recompute(m, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        ctx, _ = packed_ctx([len(toks)], m.device)
        with torch.no_grad():
            h = m.hidden_states(torch.tensor(toks, device=m.device), ctx)
            toks.append(int(m.logits(h[-1:]).argmax(-1)))
    return toks[len(prompt):]


def test_latent_cache_decode_matches_recomputation():
    _check("cpu")


@pytest.mark.gpu
def test_latent_cache_decode_on_gpu():
    _check("cuda")


def _check(device):
    torch.manual_seed(0)
    arch = PRESETS["tiny_mla_moe"]()
    m = CausalLM(arch, device=device).init_weights(7, std=0.08)
    prompts = [torch.randint(0, 500, (n,)).tolist() for n in (3, 17, 40)]
    want = [_greedy_by_recompute(m, p, 8) for p in prompts]
    for kw in (dict(), dict(max_num_batched_tokens=16)):          # whole prompts; prompts fed in chunks
        eng = RolloutEngine(m, max_model_len=128, block_size=8, num_blocks=32, **kw)
        outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
        assert [s.output for s in outs] == want, kw
        # one compressed row per token: latent rank + rotary dims, a single shared "head"
        assert eng.k_cache[0].shape[-2:] == (1, arch.kv_lora_rank + arch.qk_rope_head_dim)
        assert eng.kv_bytes_per_block() == arch.num_hidden_layers * 8 * (arch.kv_lora_rank + arch.qk_rope_head_dim) * 4


@pytest.mark.gpu
def test_latent_cache_decode_in_captured_steps():
    """bf16 weights: decode steps are captured in CUDA graphs; the latent attention has no host synchronisation."""
    torch.manual_seed(0)
    arch = PRESETS["tiny_mla_moe"]()
    m = CausalLM(arch, dtype=torch.bfloat16, device="cuda").init_weights(7, std=0.08)
    prompts = [torch.randint(0, 500, (n,)).tolist() for n in (3, 17, 40)]
    outs = {}
    for graphs in (True, False):
        eng = RolloutEngine(m, max_model_len=128, block_size=16, num_blocks=32, use_cuda_graphs=graphs)
        seqs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
        outs[graphs] = [s.output for s in seqs]
        assert bool(eng._graphs) == graphs
    assert outs[True] == outs[False]
