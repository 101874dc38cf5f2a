"""GRPO on a vision-language model end to end (CPU/gloo, world_size 2): images are preprocessed by the
prompt pipeline, generated over by the rollout engine, scored and trained on with a frozen vision tower."""
import json

from tests.dist_utils import run_ranks

SCRIPT = r'''
import os, json, time, io, torch
import numpy as np
from PIL import Image
from chatlearn_b200.algorithm.grpo import GrpoAlgorithm, GrpoConfig
from chatlearn_b200.configs import to_dataclass, resolve
from chatlearn_b200.data.synthetic import write_jsonl

out = os.environ["OUT_DIR"]
data = os.path.join(out, "train.jsonl")
if int(os.environ["RANK"]) == 0:
    rng = np.random.default_rng(0)
    rows = []
    for i in range(8):
        img = Image.fromarray(rng.integers(0, 255, (40 + 7 * i, 60 + 5 * i, 3), dtype=np.uint8))
        buf = io.BytesIO(); img.save(buf, format="PNG")
        ids = [5 + i, 6, 1002, 1000, 1003] + rng.integers(0, 900, 6).tolist()      # one placeholder per image
        rows.append({"data_source": "synthetic:mod7", "input_ids": ids, "images": [buf.getvalue().hex()],
                     "reward_model": {"ground_truth": ""}})
        if os.environ.get("VIDEO", "0") == "1" and i % 2:
            # every other record also shows a three-frame clip in front of its image
            frames = []
            for _ in range(3):
                fb = io.BytesIO(); Image.fromarray(rng.integers(0, 255, (44, 58, 3), dtype=np.uint8)).save(fb, format="PNG")
                frames.append(fb.getvalue().hex())
            rows[-1]["videos"] = [{"frames": frames, "fps": 2.0}]
            rows[-1]["input_ids"] = [7, 1002, 1001, 1003] + ids
    if os.environ.get("AGENT", "0") == "1":
        # agent task: raw chat messages, the image rides on the record and is fed to the engine by the chat model
        for i, r in enumerate(rows):
            r.pop("input_ids")
            r.update(agent_name="geo3k_agent", prompt=[{"role": "user", "content": f"what is the area of figure {i}?"}],
                     reward_model={"ground_truth": str(i)})
    write_jsonl(rows, data + ".tmp"); os.replace(data + ".tmp", data)
while not os.path.exists(data): time.sleep(0.05)
arch = {"preset": "tiny_qwen2_5_vl"}
cfg = {
  "runtime_args": {"train_backend": "fsdp", "exp_name": "vl", "output_dir": out, "data_path": data, "model_type": "vlm",
     "colocation": ["policy", "policy_trainer", "ref_policy"], "num_episode": 2, "sample_per_episode": 16,
     "train_micro_batch_size": 4, "train_global_batch_size": 16, "num_inference_per_prompt": 2,
     "save_episode_interval": 0, "max_replay_episode": 2, "log_args_dict": {"log_dir": out}},
  "models": {
    "policy_trainer": {"num_gpu": 2, "fsdp_size": 2, "trainable": True, "generation_batch_size": 8, "model_arch": arch,
       "kl_coef": 0.001, "optimizer": {"lr": 1e-4}, "packing": True, "max_token_in_packing": 512, "save_hf": False},
    "ref_policy": {"num_gpu": 2, "fsdp_size": 2, "generation_batch_size": 8, "model_arch": arch,
       "packing": True, "max_token_in_packing": 512},
    "policy": {"num_gpu": 2, "generation_batch_size": 16, "model_arch": arch, "num_inference_per_prompt": 2,
       "max_prompt_tokens_length": 128, "max_response_tokens_length": 8, "seq_length": 256, "temperature": 1.0,
       "kv_block_size": 8, "num_kv_blocks": 512, "ignore_eos": True, "max_pixels": 28 * 28 * 16,
       "tensor_model_parallel_size": int(os.environ.get("ROLLOUT_TP", "1"))},
    "reward": {"num_cpu": 2},
  }}
train_tower = os.environ.get("TRAIN_TOWER", "0") == "1"
if os.environ.get("AGENT", "0") == "1":
    cfg["runtime_args"].update(task_type="agent", use_rollout_manager=True, raw_chat=True, data_rerank=False)
    cfg["models"]["rollout_manager"] = {"num_cpu": 1, "max_concurrent_per_engine": 8}
    cfg["models"]["policy"]["tokenizer"] = "byte"
if os.environ.get("BACKEND", "fsdp") == "megatron":
    # Megatron-style trainer: tensor or pipeline parallel over the two ranks
    par = {"tensor_model_parallel_size": int(os.environ.get("TP", "1")), "pipeline_model_parallel_size": int(os.environ.get("PP", "1"))}
    mcfg = {"num_layers": 1, "hidden_size": 8, "num_attention_heads": 1, "ffn_hidden_size": 8, "max_position_embeddings": 64, "kv_channels": 8}
    cfg["runtime_args"]["train_backend"] = "megatron"
    for role in ("policy_trainer", "ref_policy"):
        cfg["models"][role].pop("fsdp_size")
        cfg["models"][role].update(par, megatron_model_cfg=dict(mcfg))
cfg["models"]["policy_trainer"]["train_vision_tower"] = train_tower
cfg = to_dataclass(GrpoConfig, resolve(cfg))
algo = GrpoAlgorithm(cfg); algo.validate()
from chatlearn_b200.models.nn.vision import build_vision_tower
from chatlearn_b200.models.nn import PRESETS
w0 = build_vision_tower(PRESETS["tiny_qwen2_5_vl"](), torch.float32, "cpu").params      # the seeded initial tower
stats = algo.run()
eng = algo.engine
tr = eng.named_models["policy_trainer"]
pol = eng.named_models["policy"]
ds = getattr(pol, "_all_datasets", None)
sample_tokens = [len(s["input_ids"]) for s in ds[0].data if "input_ids" in s] if ds else []
img_rows = getattr(pol.engine, "_image_rows_seen", 0)
# the rollout tower against the initial one and against the trainer's (its fp32 master weights after the last step
# are what the last weight sync delivered when another episode follows; compare with the bf16/fp32 working copy)
name = "visual.blocks.0.attn.qkv.weight"
moved = float((pol.engine.vision.params[name].float() - w0[name].float()).abs().max())
print("RESULT " + json.dumps({"rank": int(os.environ["RANK"]), "episodes": len(stats), "train_iters": tr._train_iteration,
      "has_tower": tr.vision is not None and pol.engine.vision is not None, "prompt_lens": sample_tokens[:3],
      "image_rows": img_rows, "tower_moved": moved, "tower_block": "vision" in tr.model.block_by_name and "vision" in pol.model.block_by_name}))
'''


def test_vision_tower_is_trained_and_synchronised(tmp_path):
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "TRAIN_TOWER": "1"})
    res = [json.loads(line[7:]) for o in outs for line in o.splitlines() if line.startswith("RESULT ")]
    assert len(res) == 2
    for r in res:
        assert r["episodes"] == 2 and r["train_iters"] == 2 and r["tower_block"]
        assert r["tower_moved"] > 0                           # the rollout engine's tower received updated weights


def test_vision_language_grpo(tmp_path):
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path)})
    res = [json.loads(line[7:]) for o in outs for line in o.splitlines() if line.startswith("RESULT ")]
    assert len(res) == 2
    for r in res:
        assert r["episodes"] == 2 and r["train_iters"] == 2 and r["has_tower"]
        assert all(n > 11 for n in r["prompt_lens"])          # the single placeholder was expanded to the image's tokens
        assert r["tower_moved"] == 0 and not r["tower_block"]  # frozen tower


def test_vision_language_grpo_with_video_clips(tmp_path):
    """Half of the records carry a clip of three frames in front of their image: preprocessing (temporal groups of two
    frames), rollout (one tensor-parallel replica over the two ranks), scoring and training with the video rows of the
    tower's output and their temporal positions."""
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "VIDEO": "1", "ROLLOUT_TP": "2"})
    res = [json.loads(line[7:]) for o in outs for line in o.splitlines() if line.startswith("RESULT ")]
    assert len(res) == 2
    for r in res:
        assert r["episodes"] == 2 and r["train_iters"] == 2 and r["has_tower"]
        assert max(r["prompt_lens"]) > min(r["prompt_lens"]) + 8        # the clips' tokens


def test_vision_language_grpo_megatron_backend(tmp_path):
    """Tensor-parallel and pipeline-parallel trainers: the first stage runs the tower, every stage gets the
    (time, row, column) positions; with a trained tower the rollout engine receives it from the first stage."""
    for name, env in (("tp2", dict(TP="2")), ("pp2", dict(PP="2", TRAIN_TOWER="1"))):
        d = tmp_path / name
        d.mkdir()
        outs, _ = run_ranks(SCRIPT, 2, env=dict(env, OUT_DIR=str(d), BACKEND="megatron"))
        res = [json.loads(line[7:]) for o in outs for line in o.splitlines() if line.startswith("RESULT ")]
        assert len(res) == 2, name
        for r in res:
            assert r["episodes"] == 2 and r["train_iters"] == 2 and r["has_tower"], (name, r)
            assert (r["tower_moved"] > 0) == ("TRAIN_TOWER" in env), (name, r)


import pytest  # noqa: E402


@pytest.mark.parametrize("video", ["0", "1"])
def test_vision_language_agent_task(tmp_path, video):
    """Agent trajectories of a vision-language model: the chat model expands the image (and video) placeholders and
    hands the pixels to the engine with every turn; training then sees the same rows."""
    outs, _ = run_ranks(SCRIPT, 2, env={"OUT_DIR": str(tmp_path), "AGENT": "1", "VIDEO": video})
    res = [json.loads(line[7:]) for o in outs for line in o.splitlines() if line.startswith("RESULT ")]
    assert len(res) == 2
    for r in res:
        assert r["episodes"] == 2 and r["train_iters"] == 2 and r["has_tower"]
        assert r["image_rows"] > 0                            # the engine embedded image patches during generation
