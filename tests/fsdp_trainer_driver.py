"""Runs one forward_step + one train_step of the data-parallel ("fsdp") trainer on a fixed batch and saves the
result (used by test_fsdp_trainer_cpu.py; one process per rank)."""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

torch.set_num_threads(1)      # fixed reduction order: runs are comparable across machine load

from chatlearn_b200.algorithm.grpo import GrpoConfig  # noqa: E402
from chatlearn_b200.checkpoint.safetensors_io import save_hf_checkpoint  # noqa: E402
from chatlearn_b200.configs import resolve, to_dataclass  # noqa: E402
from chatlearn_b200.launcher.initialize import init  # noqa: E402
from chatlearn_b200.models.nn import PRESETS, CausalLM  # noqa: E402

out = os.environ["OUT_DIR"]
tag = os.environ["TAG"]
W = int(os.environ.get("WORLD_SIZE", "1"))
rank = int(os.environ.get("RANK", "0"))
preset = os.environ.get("PRESET", "tiny_qwen3")
hf_dir = os.path.join(out, "hf_init")
if rank == 0 and not os.path.exists(os.path.join(hf_dir, "done")):
    a0 = PRESETS[preset]()
    for k, v in json.loads(os.environ.get("ARCH_JSON", "{}")).items():
        setattr(a0, k, v)
    if os.environ.get("AUX", "0") != "1":
        a0.router_aux_loss_coef = 0.0      # the balancing loss depends on how tokens are grouped into micro-batches
    m = CausalLM(a0, dtype=torch.float32).init_weights(7, std=0.05)
    save_hf_checkpoint(m, hf_dir, dtype=torch.float32)
    open(os.path.join(hf_dir, "done"), "w").close()
while not os.path.exists(os.path.join(hf_dir, "done")):
    time.sleep(0.05)

trainer = {"num_gpu": W, "trainable": True, "load": hf_dir, "fsdp_size": int(os.environ.get("FSDP", "-1")),
           "ulysses_sequence_parallel_size": int(os.environ.get("ULYSSES", "1")),
           "reshard_after_forward": os.environ.get("RESHARD", "0") == "1",
           "packing": True, "max_token_in_packing": 96, "generation_batch_size": 4, "kl_coef": 0.01,
           "entropy_coef": 0.001, "optimizer": {"lr": 1e-3, "clip_grad": 1.0}, "save_hf": False,
           "use_group_sequence_policy": os.environ.get("GSPO", "0") == "1",
           "train_vision_tower": os.environ.get("TRAIN_TOWER", "0") == "1"}
cfg = {
    "runtime_args": {"train_backend": "fsdp", "exp_name": tag, "output_dir": os.path.join(out, tag),
                     "data_path": "none", "num_episode": 1, "sample_per_episode": 8, "train_micro_batch_size": 2,
                     "train_global_batch_size": 8, "num_inference_per_prompt": 2, "save_episode_interval": 1,
                     "enable_resume_training": False, "log_args_dict": {"log_dir": out}},
    "models": {
        "policy_trainer": trainer,
        "ref_policy": {"num_gpu": W, "load": hf_dir},
        "policy": {"num_gpu": W, "model_arch": {"preset": preset}},
        "reward": {"num_cpu": 1},
    }}
cfg = to_dataclass(GrpoConfig, resolve(cfg))
init(cfg)
from chatlearn_b200.algorithm.grpo_utils.policy_trainer import PolicyTrainer  # noqa: E402

mod = PolicyTrainer("policy_trainer")
mod.placement = list(range(W))
mod.role_rank = rank
mod.init()
mod.model_setup()

g = torch.Generator().manual_seed(123)
arch = mod.model.arch
samples = []
for i in range(8):
    pl, rl = int(torch.randint(4, 12, (1,), generator=g)), int(torch.randint(6, 20, (1,), generator=g))
    toks = torch.randint(0, min(arch.vocab_size - 1, 900), (pl + rl,), generator=g)
    samples.append({"all_tokens": toks, "prompt_token_length": pl, "response_token_length": rl,
                    "advantages": float(torch.randn((), generator=g)), "prompt_uid": str(i // 2), "uid": i})
    if arch.vision_config is not None and i % 4 != 3:
        # vision-language rows: an image of (1, 4, 4) or (1, 4, 6) patches in the prompt (one sample in four has none;
        # the random text stays below the placeholder ids)
        grid = [1, 4, 4 + 2 * (i % 2)]
        n_tok = grid[1] * grid[2] // 4
        pdim = 3 * 2 * int(arch.vision_config["patch_size"]) ** 2
        toks = torch.cat([toks[:2], torch.tensor([1002] + [arch.image_token_id] * n_tok + [1003]), toks[2:]])
        samples[-1].update(all_tokens=toks, prompt_token_length=pl + n_tok + 2, image_grid_thw=[grid],
                           pixel_values=torch.randn(grid[1] * grid[2], pdim, generator=g))
noise = [0.05 * torch.randn(s["all_tokens"].numel() - 1, generator=g) for s in samples]
dp, dpr = mod.data_parallel_size, mod.data_parallel_rank
per = len(samples) // dp
mine = samples[dpr * per:(dpr + 1) * per]
mine_noise = noise[dpr * per:(dpr + 1) * per]
mod.forward_step(mine)
for s, nz in zip(mine, mine_noise):
    s["ref_logprobs"] = s["old_logprobs"] + nz
    s["old_logprobs"] = s["old_logprobs"] - 0.5 * nz
lp0 = {s["uid"]: s["old_logprobs"] + 0.5 * nz for s, nz in zip(mine, mine_noise)}
mod.train_step(mine)
prefix, metrics = mod.get_and_clear_metrics()
import torch.distributed as dist  # noqa: E402
parts = [None] * W
if W > 1:
    dist.all_gather_object(parts, lp0)
else:
    parts = [lp0]
if mod.resharded:
    with mod.state.all_gathered() as whole:          # (a collective: every rank)
        sd = {k: v.float().clone() for k, v in whole.hf_state_dict().items()}
else:
    sd = {k: v.float() for k, v in mod.model.hf_state_dict().items()}
if rank == 0:
    lps = {u: v for p in parts for u, v in p.items()}
    torch.save({"sd": sd, "metrics": metrics,
                "logprobs": [lps[i] for i in range(8)]}, os.path.join(out, f"{tag}.pt"))
    print("RESULT " + json.dumps({k: float(v) for k, v in metrics.items()}))
