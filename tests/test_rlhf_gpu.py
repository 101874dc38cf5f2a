"""Actor-critic RLHF on one B200: policy, reference, reward and value roles with Llama-2-7B layer shapes (two layers
each), bf16, this package's kernels.  Two episodes must train both the policy and the critic."""
import json
import os
import subprocess
import sys

import pytest
import torch

from chatlearn_b200.utils.utils import get_free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import os, json, sys, torch
sys.path.insert(0, os.environ["REPO_ROOT"])
from chatlearn_b200 import ops
from chatlearn_b200.algorithm.rlhf import RlhfAlgorithm, RlhfConfig
from chatlearn_b200.configs import to_dataclass, resolve
from chatlearn_b200.data.synthetic import make_prompts, write_jsonl

out = os.environ["OUT_DIR"]
data = os.path.join(out, "train.jsonl")
arch = {"preset": "llama2_7b", "num_hidden_layers": 2}
write_jsonl(make_prompts(32, 32, 128, 32000, seed=0, data_source="synthetic:rm"), data)
tr = {"num_gpu": 1, "fsdp_size": 1, "trainable": True, "generation_batch_size": 16, "model_arch": arch,
      "kl_coef": 0.0, "optimizer": {"lr": 1e-5}, "packing": True, "max_token_in_packing": 4096, "save_hf": False,
      "gradient_checkpointing": False}
cfg = {
  "runtime_args": {"train_backend": "fsdp", "exp_name": "rlhf", "output_dir": out, "data_path": data,
     "colocation": ["policy", "policy_trainer", "reference", "reward", "value_trainer"],
     "num_episode": 2, "sample_per_episode": 32, "train_micro_batch_size": 8, "train_global_batch_size": 32,
     "num_inference_per_prompt": 1, "save_episode_interval": 0, "log_args_dict": {"log_dir": out}},
  "models": {
    "policy_trainer": dict(tr),
    "value_trainer": dict(tr, seed=99),
    "reference": {"num_gpu": 1, "fsdp_size": 1, "generation_batch_size": 16, "model_arch": arch},
    "reward": {"num_gpu": 1, "fsdp_size": 1, "generation_batch_size": 16, "model_arch": arch, "seed": 77,
               "clip_reward_value": 5.0},
    "policy": {"num_gpu": 1, "generation_batch_size": 32, "model_arch": arch, "num_inference_per_prompt": 1,
       "max_prompt_tokens_length": 130, "max_response_tokens_length": 64, "temperature": 1.0, "kv_block_size": 64,
       "num_kv_blocks": 256, "ignore_eos": True},
  }}
cfg = to_dataclass(RlhfConfig, resolve(cfg))
algo = RlhfAlgorithm(cfg); algo.validate()
eng = algo.run()
print("RESULT " + json.dumps({"episodes": len(eng.episode_stats), "train_iters": eng.named_models["policy_trainer"]._train_iteration,
      "critic_iters": eng.named_models["value_trainer"]._train_iteration,
      "launches": int(sum(ops.launch_counts.values())), "device": str(eng.named_models["policy_trainer"].device)}))
'''


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_actor_critic_rlhf_on_one_gpu(tmp_path):
    script = tmp_path / "rlhf_gpu.py"
    script.write_text(SCRIPT)
    env = dict(os.environ, OUT_DIR=str(tmp_path), REPO_ROOT=ROOT, RANK="0", LOCAL_RANK="0", WORLD_SIZE="1",
               MASTER_ADDR="127.0.0.1", MASTER_PORT=str(get_free_port()))
    env.pop("CHATLEARN_FORCE_CPU", None)
    p = subprocess.run([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=600)
    assert p.returncode == 0, p.stdout[-3000:]
    res = [json.loads(line[7:]) for line in p.stdout.splitlines() if line.startswith("RESULT ")]
    assert len(res) == 1, p.stdout[-2000:]
    r = res[0]
    assert r["episodes"] == 2 and r["train_iters"] == 2 and r["critic_iters"] == 2
    assert r["device"].startswith("cuda") and r["launches"] > 100
    lines = [json.loads(x) for x in open(tmp_path / "metrics.jsonl")]
    assert any(any(k.endswith("rm_score") for k in l) for l in lines)
