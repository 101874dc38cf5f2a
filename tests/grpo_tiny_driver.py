"""Tiny GRPO job used by the tests (run as a script, one process per rank)."""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from chatlearn_b200 import ops  # noqa: E402
from chatlearn_b200.algorithm.grpo import GrpoAlgorithm, GrpoConfig  # noqa: E402
from chatlearn_b200.configs import resolve, to_dataclass  # noqa: E402
from chatlearn_b200.data.synthetic import make_prompts, write_jsonl  # noqa: E402

out = os.environ["OUT_DIR"]
world = int(os.environ.get("WORLD_SIZE", "1"))
data = os.path.join(out, "train.jsonl")
if int(os.environ.get("RANK", "0")) == 0:
    write_jsonl(make_prompts(8, 16, 48, 1024, seed=0, data_source="synthetic:mod7"), data + ".tmp")
    os.replace(data + ".tmp", data)
while not os.path.exists(data):
    time.sleep(0.05)
arch = {"preset": os.environ.get("PRESET", "tiny_qwen3")}
cfg = {
    "runtime_args": {"train_backend": "fsdp", "exp_name": "tiny", "colocation": ["policy", "policy_trainer", "ref_policy"],
                     "output_dir": out, "data_path": data, "num_episode": 2, "sample_per_episode": 32,
                     "train_micro_batch_size": 4, "train_global_batch_size": 32, "num_inference_per_prompt": 4,
                     "save_episode_interval": 100, "max_replay_episode": 2, "log_args_dict": {"log_dir": out}},
    "models": {
        "policy_trainer": {"num_gpu": world, "fsdp_size": world, "trainable": True, "generation_batch_size": 8,
                           "model_arch": arch, "kl_coef": 0.001, "optimizer": {"lr": 1e-5}, "packing": True,
                           "max_token_in_packing": 256, "save_hf": False,
                           "free_gpu_memory": {"offload_weights": True, "offload_optimizer_states": True,
                                               "free_grad_buffers": True}},
        "ref_policy": {"num_gpu": world, "fsdp_size": world, "generation_batch_size": 8, "model_arch": arch,
                       "packing": True, "max_token_in_packing": 256, "free_gpu_memory": {"offload_weights": True}},
        "policy": {"num_gpu": world, "tensor_model_parallel_size": int(os.environ.get("TP", "1")),
                   "generation_batch_size": 16, "model_arch": arch, "num_inference_per_prompt": 4,
                   "max_prompt_tokens_length": 64, "max_response_tokens_length": 32, "kv_block_size": 16,
                   "num_kv_blocks": 256, "ignore_eos": True},
        "reward": {"num_cpu": world},
    }}
cfg = to_dataclass(GrpoConfig, resolve(cfg))
algo = GrpoAlgorithm(cfg)
algo.validate()
stats = algo.run()
eng = algo.engine
pol, tr = eng.named_models["policy"], eng.named_models["policy_trainer"]
tr.onload(to_onload_weights=True, to_build_grad_buffers=False, to_onload_optimizer_states=False)
sd_t, sd_p = tr.model.hf_state_dict(), pol.model.hf_state_dict()
maxdiff = 0.0
for k, v in sd_p.items():
    nz = v != 0
    if nz.any():
        maxdiff = max(maxdiff, (v.float() - sd_t[k].float())[nz].abs().max().item())
print("RESULT " + json.dumps({"episodes": len(stats), "maxdiff": maxdiff,
                              "native_launches": int(sum(ops.launch_counts.values())),
                              "library_calls": dict(ops.library_counts)}))
