"""GRPO end to end with the tensor-parallel ("megatron") trainer backend on CPU/gloo, world_size 2:
TP=2 trainer and reference, two rollout replicas, TP-sharded → whole weight resharding every episode."""
import json

from tests.dist_utils import run_ranks

SCRIPT = r'''
import os, json, time, torch
from chatlearn_b200.algorithm.grpo import GrpoAlgorithm, GrpoConfig
from chatlearn_b200.configs import to_dataclass, resolve
from chatlearn_b200.data.synthetic import make_prompts, write_jsonl

out = os.environ["OUT_DIR"]
data = os.path.join(out, "train.jsonl")
if int(os.environ["RANK"]) == 0:
    write_jsonl(make_prompts(8, 8, 24, 256, seed=0, data_source="synthetic:mod7"), data + ".tmp")
    os.replace(data + ".tmp", data)
while not os.path.exists(data): time.sleep(0.05)
arch = {"preset": os.environ.get("PRESET", "tiny_qwen3")}
mcfg = {"num_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "ffn_hidden_size": 704,
        "max_position_embeddings": 512, "kv_channels": 64}
par = {"tensor_model_parallel_size": int(os.environ.get("TP", "2")), "pipeline_model_parallel_size": int(os.environ.get("PP", "1")),
       "context_parallel_size": int(os.environ.get("CP", "1")), "expert_model_parallel_size": int(os.environ.get("EP", "1")),
       "virtual_pipeline_model_parallel_size": int(os.environ.get("VPP", "1"))}
cfg = {
  "runtime_args": {"train_backend": "megatron", "exp_name": "mg", "output_dir": out, "data_path": data,
     "colocation": ["policy", "policy_trainer", "ref_policy"], "num_episode": 2, "sample_per_episode": 16,
     "train_micro_batch_size": 4, "train_global_batch_size": 16, "num_inference_per_prompt": 2,
     "save_episode_interval": 2, "max_replay_episode": 2, "log_args_dict": {"log_dir": out}},
  "models": {
    "policy_trainer": dict(par, num_gpu=2, trainable=True, generation_batch_size=8, model_arch=arch, kl_coef=0.001,
       optimizer={"lr": 1e-4}, packing=True, max_token_in_packing=256, megatron_model_cfg=dict(mcfg),
       max_prompt_tokens_length=64, max_response_tokens_length=16),
    "ref_policy": dict(par, num_gpu=2, generation_batch_size=8, model_arch=arch, packing=True, max_token_in_packing=256,
       megatron_model_cfg=dict(mcfg), max_prompt_tokens_length=64, max_response_tokens_length=16),
    "policy": {"num_gpu": 2, "generation_batch_size": 16, "model_arch": arch, "num_inference_per_prompt": 2,
       "max_prompt_tokens_length": 64, "max_response_tokens_length": 16, "seq_length": 128, "temperature": 1.0,
       "kv_block_size": 8, "num_kv_blocks": 256, "ignore_eos": True,
       "expert_model_parallel_size": int(os.environ.get("ROLLOUT_EP", "1")),
       "tensor_model_parallel_size": int(os.environ.get("ROLLOUT_TP", "1"))},
    "reward": {"num_cpu": 2},
  }}
cfg = to_dataclass(GrpoConfig, resolve(cfg))
algo = GrpoAlgorithm(cfg); algo.validate()
stats = algo.run()
eng = algo.engine
tr, pol = eng.named_models["policy_trainer"], eng.named_models["policy"]
tr.onload()
# the rollout copy equals the trainer's shards put back together: compare this rank's shard of every HF tensor
sd_p = pol.model.hf_state_dict()
sd_t = tr.model.hf_state_dict()
maxdiff = 0.0
for k, v in sd_t.items():
    nz = v != 0
    if nz.any():
        maxdiff = max(maxdiff, (sd_p[k].to(v.dtype) - v)[nz].abs().max().item())
print("RESULT " + json.dumps({"rank": int(os.environ["RANK"]), "episodes": len(stats), "maxdiff": maxdiff,
      "train_iters": tr._train_iteration}))
'''


def _res(outs):
    return [json.loads(line[7:]) for o in outs for line in o.splitlines() if line.startswith("RESULT ")]


def test_grpo_tp2_trainer(tmp_path):
    res = _res(run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path)})[0])
    assert len(res) == 2 and all(r["episodes"] == 2 and r["train_iters"] == 2 and r["maxdiff"] == 0.0 for r in res)
    assert (tmp_path / "save_model" / "policy_trainer").exists()


def test_grpo_pp2_trainer(tmp_path):
    res = _res(run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "TP": "1", "PP": "2"})[0])
    assert len(res) == 2 and all(r["episodes"] == 2 and r["maxdiff"] == 0.0 for r in res)


def test_grpo_moe_ep2_trainer_and_ep2_rollout(tmp_path):
    """Expert-parallel trainer (experts re-homed over two ranks) feeding an expert-parallel rollout."""
    env = {"OUT_DIR": str(tmp_path), "PRESET": "tiny_moe", "TP": "1", "EP": "2", "ROLLOUT_EP": "2"}
    res = _res(run_ranks(SCRIPT, 2, env=env)[0])
    assert len(res) == 2 and all(r["episodes"] == 2 and r["train_iters"] == 2 and r["maxdiff"] == 0.0 for r in res)


def test_grpo_mla_moe_cp2_trainer(tmp_path):
    """MLA attention + sigmoid-routed MoE with context parallelism 2 in the trainer."""
    env = {"OUT_DIR": str(tmp_path), "PRESET": "tiny_mla_moe", "TP": "1", "CP": "2"}
    res = _res(run_ranks(SCRIPT, 2, env=env)[0])
    assert len(res) == 2 and all(r["episodes"] == 2 and r["maxdiff"] == 0.0 for r in res)


def test_grpo_qwen3_next_pp2_trainer(tmp_path):
    """Gated delta-net hybrid under the Megatron-style trainer: two pipeline stages (two layers each); the
    rollout weights equal the trainer's after the last sync."""
    res = _res(run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "TP": "1", "PP": "2", "PRESET": "tiny_qwen3_next"})[0])
    assert len(res) == 2 and all(r["episodes"] == 2 and r["maxdiff"] == 0.0 for r in res)


def test_grpo_pp2_with_two_model_chunks_per_stage(tmp_path):
    """Interleaved pipeline schedule end to end: four layers as 2 stages x 2 chunks (stage 0 holds layers 0 and 2),
    scoring, training, checkpoint, and a weight sync that leaves the rollout weights equal to the trainer's."""
    res = _res(run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "TP": "1", "PP": "2", "VPP": "2",
                                         "PRESET": "tiny_qwen3_next"})[0])
    assert len(res) == 2 and all(r["episodes"] == 2 and r["maxdiff"] == 0.0 for r in res)


def test_grpo_qwen3_next_tensor_parallel(tmp_path):
    """Gated delta-net hybrid with the heads of both mixer kinds split over two tensor-parallel ranks, in the trainer
    (sequence-parallel rows between the layers) and in the rollout engine (recurrent state of this rank's heads):
    after the last sync every rank's rollout shard equals the trainer's."""
    res = _res(run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "TP": "2", "PP": "1", "ROLLOUT_TP": "2",
                                         "PRESET": "tiny_qwen3_next"})[0])
    assert len(res) == 2 and all(r["episodes"] == 2 and r["maxdiff"] == 0.0 for r in res)
