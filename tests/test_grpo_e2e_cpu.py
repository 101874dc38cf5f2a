"""End-to-end GRPO on CPU/gloo, world_size 2: tiny Qwen3, synthetic prompts,
mod-7 reward, full weight sync into the rollout engine every iteration."""
import json
import os

from tests.dist_utils import run_ranks

SCRIPT = r'''
import os, json, tempfile, torch
from chatlearn_b200.algorithm.grpo import GrpoAlgorithm, GrpoConfig
from chatlearn_b200.configs import to_dataclass, resolve
from chatlearn_b200.data.synthetic import make_prompts, write_jsonl

out = os.environ["OUT_DIR"]
data = os.path.join(out, "train.jsonl")
if int(os.environ["RANK"]) == 0:
    write_jsonl(make_prompts(8, 16, 48, 1024, seed=0, data_source="synthetic:mod7"), data)
cfg = {
  "runtime_args": {"train_backend": "fsdp", "rollout_backend": "native", "exp_name": "tiny",
     "colocation": ["policy", "policy_trainer", "ref_policy"], "output_dir": out, "data_path": data,
     "data_checkpoint_path": out + "/data_ckpt", "num_episode": int(os.environ.get("EPISODES", "2")),
     "sample_per_episode": 32, "train_micro_batch_size": 4, "train_global_batch_size": 32,
     "num_inference_per_prompt": 4, "save_episode_interval": 1, "max_replay_episode": 2,
     "bucket_size_mb_in_memory_manager": float(os.environ.get("SYNC_BUCKET_MB", "1024")),
     "log_args_dict": {"log_dir": out}},
  "models": {
    "policy_trainer": {"num_gpu": 2, "fsdp_size": int(os.environ.get("FSDP_SIZE", "2")), "trainable": True, "generation_batch_size": 8,
       "model_arch": {"preset": "tiny_qwen3"}, "kl_coef": 0.001, "optimizer": {"lr": 1e-5},
       "reshard_after_forward": os.environ.get("RESHARD", "0") == "1",
       "packing": os.environ.get("PACKING", "0") == "1", "max_token_in_packing": 256, "save_hf": True,
       "free_gpu_memory": {"offload_weights": True, "offload_optimizer_states": os.environ.get("REGEN", "0") != "1",
                           "free_grad_buffers": True}},
    "ref_policy": {"num_gpu": 2, "fsdp_size": 2, "generation_batch_size": 8, "model_arch": {"preset": "tiny_qwen3"},
       "free_gpu_memory": {"offload_weights": True}},
    "policy": {"num_gpu": 2, "tensor_model_parallel_size": int(os.environ.get("TP", "1")), "generation_batch_size": 16,
       "model_arch": {"preset": "tiny_qwen3"}, "num_inference_per_prompt": 4, "max_prompt_tokens_length": 64,
       "max_response_tokens_length": 32, "temperature": 1.0, "kv_block_size": 8, "num_kv_blocks": 256,
       "ignore_eos": True},
    "reward": {"num_cpu": 2},
  }}
import time
while not os.path.exists(data): time.sleep(0.05)
cfg = to_dataclass(GrpoConfig, resolve(cfg))
algo = GrpoAlgorithm(cfg); algo.validate()
stats = algo.run()
eng = algo.engine
pol, tr = eng.named_models["policy"], eng.named_models["policy_trainer"]
# after the final sync the rollout weights equal the trainer weights
tr.onload()
if os.environ.get("RESHARD", "0") == "1":
    with tr.state.all_gathered():
        sd_t = {k: v.clone() for k, v in tr.model.hf_state_dict().items()}
else:
    sd_t = tr.model.hf_state_dict()
sd_p = pol.model.hf_state_dict()
maxdiff = 0.0
for k, v in sd_p.items():
    nz = v != 0
    maxdiff = max(maxdiff, (v - sd_t[k])[nz].abs().max().item() if nz.any() else 0.0)
print("RESULT " + json.dumps({"rank": int(os.environ["RANK"]), "episodes": len(stats), "maxdiff": maxdiff,
      "iters": eng.trainer.iteration, "consumed": cfg.runtime_args.consumed_samples,
      "tps": stats[-1].get("tps_throughput", 0),
      "sync_iterations": max(g.stats.get("iterations", 0) for g in eng.model_manager.parameter_sync_groups.values())}))
'''


def _results(outs):
    res = []
    for o in outs:
        for line in o.splitlines():
            if line.startswith("RESULT "):
                res.append(json.loads(line[7:]))
    return res


def test_grpo_tiny_gloo_ws2(tmp_path):
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path)})
    res = _results(outs)
    assert len(res) == 2
    for r in res:
        assert r["episodes"] == 2 and r["iters"] == 2 and r["consumed"] == 64
        assert r["maxdiff"] == 0.0
    # checkpoints in the reference layout
    assert os.path.exists(tmp_path / "data_ckpt" / "latest_checkpointed_iteration.txt")
    d = tmp_path / "save_model" / "policy_trainer" / "2"
    assert (d / "model_world_size_2_rank_0.pt").exists() and (d / "optim_world_size_2_rank_1.pt").exists()
    assert (d / "huggingface" / "model.safetensors").exists()
    assert (tmp_path / "metrics.jsonl").exists()
    # the engine that generated the tokens and the trainer agree on their log-probabilities (fp32 on CPU)
    diffs = [v for line in open(tmp_path / "metrics.jsonl") for k, v in json.loads(line).items()
             if k.endswith("rollout_logprob_abs_diff_max")]
    assert diffs and max(diffs) < 1e-4, diffs


def test_grpo_tiny_packing_tp2(tmp_path):
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "PACKING": "1", "TP": "2", "EPISODES": "1"})
    res = _results(outs)
    assert len(res) == 2 and all(r["maxdiff"] == 0.0 for r in res)


def test_weight_sync_in_memory_budgeted_iterations(tmp_path):
    """Parameter-sharded trainer (every rank holds half of each block, so the rollout ranks pull remote pieces),
    messages capped at 16 KB: the point-to-point weight sync runs as several planned iterations and the rollout
    weights still equal the trainer's."""
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "TP": "2", "EPISODES": "1", "SYNC_BUCKET_MB": "0.015625",
                                        "RESHARD": "1"})
    res = _results(outs)
    assert len(res) == 2 and all(r["maxdiff"] == 0.0 for r in res)
    assert all(r["sync_iterations"] > 1 for r in res), res


def test_hybrid_sharding_two_replicas_of_one(tmp_path):
    """``fsdp_size`` 1 on two GPUs: every rank is its own shard group and the two all-reduce their gradients."""
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "EPISODES": "1", "FSDP_SIZE": "1"})
    res = _results(outs)
    assert len(res) == 2 and all(r["episodes"] == 1 and r["maxdiff"] == 0.0 for r in res)


def test_resume_continues_from_checkpoint(tmp_path):
    """One episode with checkpoints, then a fresh job over the same output directory: it resumes the data
    position and the trainer state and runs only the remaining episode."""
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "EPISODES": "1"})
    first = _results(outs)
    assert all(r["episodes"] == 1 and r["consumed"] == 32 for r in first)
    outs, logs = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "EPISODES": "2"})
    second = _results(outs)
    assert len(second) == 2
    for r in second:
        assert r["episodes"] == 1, "only the second episode runs after the resume"
        assert r["consumed"] == 64 and r["maxdiff"] == 0.0
    assert (tmp_path / "save_model" / "policy_trainer" / "2").exists()


def test_trainer_weights_dropped_and_rebuilt_from_master(tmp_path):
    """With the optimizer state resident, the trainer's compute-dtype weights are dropped during rollout and
    rebuilt from the fp32 master shards (cast + all-gather): the run must be indistinguishable."""
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "REGEN": "1"})
    res = _results(outs)
    assert len(res) == 2 and all(r["episodes"] == 2 and r["maxdiff"] == 0.0 for r in res)
