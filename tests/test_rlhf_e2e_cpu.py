"""RLHF recipes end to end on CPU/gloo (world_size 2): three-model and actor-critic."""
import json

from tests.dist_utils import run_ranks

SCRIPT = r'''
import os, json, time, torch
from chatlearn_b200.algorithm.rlhf import RlhfAlgorithm, RlhfConfig
from chatlearn_b200.configs import to_dataclass, resolve
from chatlearn_b200.data.synthetic import make_prompts, write_jsonl

out = os.environ["OUT_DIR"]
data = os.path.join(out, "train.jsonl")
if int(os.environ["RANK"]) == 0:
    write_jsonl(make_prompts(8, 8, 24, 512, seed=0, data_source="synthetic:rm"), data)
while not os.path.exists(data): time.sleep(0.05)
arch = {"preset": "tiny_llama"}
critic = os.environ.get("CRITIC", "0") == "1"
n = 1 if critic else 2
tr = {"num_gpu": 2, "fsdp_size": 2, "trainable": True, "generation_batch_size": 8, "model_arch": arch,
      "kl_coef": 0.0, "optimizer": {"lr": 1e-4}, "packing": True, "max_token_in_packing": 256, "save_hf": False,
      "gradient_checkpointing": False}
cfg = {
  "runtime_args": {"train_backend": "fsdp", "exp_name": "rlhf", "output_dir": out, "data_path": data,
     "colocation": ["policy", "policy_trainer", "reference", "reward"] + (["value_trainer"] if critic else []),
     "num_episode": 2, "sample_per_episode": 16, "train_micro_batch_size": 4, "train_global_batch_size": 16,
     "num_inference_per_prompt": n, "save_episode_interval": 0, "log_args_dict": {"log_dir": out}},
  "models": {
    "policy_trainer": dict(tr),
    "reference": {"num_gpu": 2, "fsdp_size": 2, "generation_batch_size": 8, "model_arch": arch},
    "reward": {"num_gpu": 2, "fsdp_size": 2, "generation_batch_size": 8, "model_arch": arch, "seed": 77,
               "clip_reward_value": 5.0},
    "policy": {"num_gpu": 2, "generation_batch_size": 16, "model_arch": arch, "num_inference_per_prompt": n,
       "max_prompt_tokens_length": 32, "max_response_tokens_length": 16, "temperature": 1.0, "kv_block_size": 8,
       "num_kv_blocks": 128, "ignore_eos": True},
  }}
if critic:
    cfg["models"]["value_trainer"] = dict(tr, seed=99)
cfg = to_dataclass(RlhfConfig, resolve(cfg))
algo = RlhfAlgorithm(cfg); algo.validate()
eng = algo.run()
st = eng.episode_stats
tr_m = eng.named_models["policy_trainer"]
res = {"rank": int(os.environ["RANK"]), "episodes": len(st), "iters": eng.trainer.iteration,
       "train_iters": tr_m._train_iteration}
if critic:
    res["critic_iters"] = eng.named_models["value_trainer"]._train_iteration
print("RESULT " + json.dumps(res))
'''


def _results(outs):
    return [json.loads(line[7:]) for o in outs for line in o.splitlines() if line.startswith("RESULT ")]


def test_three_model_rlhf(tmp_path):
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path)})
    res = _results(outs)
    assert len(res) == 2 and all(r["episodes"] == 2 and r["train_iters"] == 2 for r in res)
    lines = [json.loads(x) for x in open(tmp_path / "metrics.jsonl")]
    assert any("reward/rm_score" in l or any(k.endswith("rm_score") for k in l) for l in lines)


def test_actor_critic_rlhf(tmp_path):
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "CRITIC": "1"})
    res = _results(outs)
    assert len(res) == 2 and all(r["train_iters"] == 2 and r["critic_iters"] == 2 for r in res)
