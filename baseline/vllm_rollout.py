"""Same-box rollout figure of the library the reference generates with.

    python baseline/vllm_rollout.py [--tp 1] [--prompts 16] [--samples 8] [--max-response 2048]

The reference's rollout role is a vLLM engine (chatlearn/models/vllm_module.py:131-216: ``LLM(...)`` with
``disable_custom_all_reduce=True``, generation through ``llm.generate``).  Its adapter pins vLLM 0.8.5 and cannot
start here; this script times the installed vLLM (0.22) alone on the rollout phase of the flagship configuration:
Qwen3-8B architecture with dummy (random) weights, the same synthetic prompts as ``bench.py`` (16 prompts of 128-1024
uniform-random tokens, 8 samples each), temperature 1, 2048 new tokens per sample with EOS ignored.  It prints one
JSON line with generated tokens per second and seconds per rollout, after one untimed warm-up rollout.  Nothing of
this package runs in it: it is the number next to ``rollout/gen_tokens_per_s`` of ``bench.py``.
"""
import argparse
import json
import os
import sys
import tempfile
import time

os.environ.setdefault("HF_HUB_OFFLINE", "1")
os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
os.environ.setdefault("DO_NOT_TRACK", "1")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--prompts", type=int, default=16)
    ap.add_argument("--samples", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, nargs=2, default=[128, 1024])
    ap.add_argument("--max-response", type=int, default=2048)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    a = ap.parse_args()
    import torch
    from transformers import Qwen3Config
    from vllm import LLM, SamplingParams

    from chatlearn_b200.data.synthetic import make_prompts
    d = tempfile.mkdtemp(prefix="qwen3_8b_dummy_")
    Qwen3Config(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False, torch_dtype="bfloat16",
                architectures=["Qwen3ForCausalLM"]).save_pretrained(d)
    llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", tensor_parallel_size=a.tp,
              gpu_memory_utilization=a.gpu_memory_utilization, max_model_len=a.prompt_len[1] + a.max_response + 8,
              max_num_seqs=256, max_num_batched_tokens=16384, disable_custom_all_reduce=True, seed=0)
    sp = SamplingParams(temperature=1.0, top_p=1.0, top_k=-1, max_tokens=a.max_response, ignore_eos=True, detokenize=False)

    def batch(seed):
        rows = make_prompts(a.prompts, a.prompt_len[0], a.prompt_len[1], 151936, seed=seed, data_source="synthetic:hash30")
        out = []
        for r in rows:
            ids = [int(t) for t in (r.get("input_ids") or r.get("prompt_token_ids") or r["prompt"])]
            out.extend([{"prompt_token_ids": ids}] * a.samples)      # the reference repeats each prompt n times
        return out

    llm.generate(batch(1), sp, use_tqdm=False)                       # warm-up: compilation, graph capture
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = llm.generate(batch(2), sp, use_tqdm=False)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    gen = sum(len(o.outputs[0].token_ids) for o in outs)
    import vllm
    print(json.dumps({"impl": f"vllm {vllm.__version__}", "model": "qwen3_8b (dummy weights)", "tp": a.tp,
                      "sequences": len(outs), "generated_tokens": gen, "rollout_s": round(dt, 3),
                      "gen_tokens_per_s": round(gen / dt, 1), "prompt_len": a.prompt_len, "max_response": a.max_response}), flush=True)


if __name__ == "__main__":
    main()
