"""GRPO variants end to end on CPU/gloo (world_size 2): partial rollout, and agent
tasks through the rollout manager."""
import json

from tests.dist_utils import run_ranks

SCRIPT = r'''
import os, json, time, torch
from chatlearn_b200.algorithm.grpo import GrpoAlgorithm, GrpoConfig
from chatlearn_b200.configs import to_dataclass, resolve
from chatlearn_b200.data.synthetic import make_prompts, write_jsonl

out, mode = os.environ["OUT_DIR"], os.environ["MODE"]
data = os.path.join(out, "train.jsonl")
if int(os.environ["RANK"]) == 0:
    if mode == "agent":
        rows = [{"data_source": "synthetic:mod7", "agent_name": "matheval_agent",
                 "prompt": [{"role": "user", "content": f"what is {i}+{i}?"}],
                 "reward_model": {"ground_truth": str(2 * i)}} for i in range(8)]
        write_jsonl(rows, data + ".tmp")
    else:
        write_jsonl(make_prompts(8, 16, 32, 512, seed=0, data_source="synthetic:mod7"), data + ".tmp")
    os.replace(data + ".tmp", data)
while not os.path.exists(data): time.sleep(0.05)
arch = {"preset": {"moe": "tiny_moe", "next": "tiny_qwen3_next"}.get(mode, "tiny_llama")}
cfg = {
  "runtime_args": {"train_backend": "fsdp", "exp_name": mode, "output_dir": out, "data_path": data,
     "colocation": ["policy", "policy_trainer", "ref_policy"],
     "num_episode": 3, "sample_per_episode": 32, "train_micro_batch_size": 4, "train_global_batch_size": 32,
     "num_inference_per_prompt": 4, "save_episode_interval": 0, "max_replay_episode": 4,
     "log_args_dict": {"log_dir": out}},
  "models": {
    "policy_trainer": {"num_gpu": 2, "fsdp_size": 2, "trainable": True, "generation_batch_size": 8, "model_arch": arch,
       "kl_coef": 0.001, "optimizer": {"lr": 1e-5}, "packing": True, "max_token_in_packing": 512, "save_hf": False},
    "ref_policy": {"num_gpu": 2, "fsdp_size": 2, "generation_batch_size": 8, "model_arch": arch},
    "policy": {"num_gpu": 2, "generation_batch_size": 16, "model_arch": arch, "num_inference_per_prompt": 4,
       "max_prompt_tokens_length": 64, "max_response_tokens_length": 16, "seq_length": 256, "temperature": 1.0,
       "kv_block_size": 8, "num_kv_blocks": 512, "ignore_eos": True, "tokenizer": "byte"},
    "reward": {"num_cpu": 2},
  }}
if mode == "moe":
    # expert-parallel rollout: each of the two ranks hosts half of the experts and decodes its own sequences
    cfg["models"]["policy"].update(expert_model_parallel_size=2, tokenizer="null")
if mode == "next":
    cfg["models"]["policy"].update(tokenizer="null")
if mode == "partial":
    cfg["runtime_args"]["use_partial_rollout"] = True
    cfg["models"]["partial_rollout_manager"] = {"num_cpu": 1, "max_rollout_round": 2, "rollout_ratio": [0.5, 0.5],
                                                "mini_response_per_prompt": 2}
if mode == "agent":
    cfg["runtime_args"].update(task_type="agent", use_rollout_manager=True, raw_chat=True, data_rerank=False)
    cfg["models"]["rollout_manager"] = {"num_cpu": 1, "max_concurrent_per_engine": 8}
cfg = to_dataclass(GrpoConfig, resolve(cfg))
algo = GrpoAlgorithm(cfg); algo.validate()
stats = algo.run()
eng = algo.engine
print("RESULT " + json.dumps({"rank": int(os.environ["RANK"]), "episodes": len(stats),
      "train_iters": eng.named_models["policy_trainer"]._train_iteration}))
'''


def _results(outs):
    return [json.loads(line[7:]) for o in outs for line in o.splitlines() if line.startswith("RESULT ")]


def _metrics(tmp_path):
    return [json.loads(x) for x in open(tmp_path / "metrics.jsonl")]


def test_partial_rollout(tmp_path):
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "MODE": "partial"})
    res = _results(outs)
    assert len(res) == 2 and all(r["episodes"] == 3 for r in res)
    keys = set().union(*[set(m) for m in _metrics(tmp_path)])
    assert any(k.endswith("round_1_samples") for k in keys) and any(k.endswith("num_train_samples") for k in keys)
    # ignore_eos: every sample uses its whole first-round budget, so it is carried into a second round
    carried = [m[k] for m in _metrics(tmp_path) for k in m if k.endswith("round_1_samples")]
    assert max(carried) > 0


def test_agent_through_rollout_manager(tmp_path):
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "MODE": "agent"})
    res = _results(outs)
    assert len(res) == 2 and all(r["episodes"] == 3 and r["train_iters"] == 3 for r in res)
    keys = set().union(*[set(m) for m in _metrics(tmp_path)])
    assert any(k.endswith("num_turns") for k in keys)


def test_moe_model_with_expert_parallel_rollout(tmp_path):
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "MODE": "moe"})
    res = _results(outs)
    assert len(res) == 2 and all(r["episodes"] == 3 and r["train_iters"] == 3 for r in res)


def test_qwen3_next_hybrid_model(tmp_path):
    """Gated delta-net + gated attention + shared-expert MoE: sharded training, weight sync into the rollout
    engine (recurrent state per sequence), three episodes."""
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "MODE": "next"})
    res = _results(outs)
    assert len(res) == 2 and all(r["episodes"] == 3 and r["train_iters"] == 3 for r in res)
    ms = [m for m in _metrics(tmp_path) if any(k.endswith("grad_norm") for k in m)]
    assert ms and all(v == v and v < 1e4 for m in ms for k, v in m.items() if k.endswith("grad_norm"))
