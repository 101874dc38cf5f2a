"""The command line: `python -m chatlearn_b200 grpo --config-file template/grpo_fsdp.yaml key=value ...`
forks two CPU ranks and runs one GRPO episode from the shipped template."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_grpo_cli_from_template(tmp_path):
    from chatlearn_b200.data.synthetic import make_prompts, write_jsonl
    data = tmp_path / "data.jsonl"
    write_jsonl(make_prompts(8, 8, 24, 1024, seed=0, data_source="synthetic:mod7"), str(data))
    arch = "{preset: tiny_qwen3}"
    cmd = [sys.executable, "-m", "chatlearn_b200", "grpo", "--nproc", "2", "--cpu", "--config-file",
           os.path.join(ROOT, "template", "grpo_fsdp.yaml"),
           f"runtime_args.data_path={data}", f"runtime_args.output_dir={tmp_path / 'out'}", "runtime_args.num_episode=1",
           "runtime_args.sample_per_episode=16", "runtime_args.train_global_batch_size=16",
           "runtime_args.train_micro_batch_size=4", "runtime_args.num_inference_per_prompt=2",
           "runtime_args.save_episode_interval=0", "runtime_args.eval_episode_interval=0",
           f"models.policy_trainer.model_arch={arch}", f"models.ref_policy.model_arch={arch}", f"models.policy.model_arch={arch}",
           "models.policy_trainer.load=null", "models.policy_trainer.num_gpu=2", "models.policy_trainer.max_token_in_packing=512",
           "models.policy.max_prompt_tokens_length=64", "models.policy.max_response_tokens_length=8",
           "models.policy.num_kv_blocks=256", "models.policy.kv_block_size=8", "models.reward.num_cpu=2",
           "models.partial_rollout_manager=null", "models.rollout_manager=null"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    out = p.stdout + p.stderr
    assert p.returncode == 0, out[-3000:]
    assert "grpo finished" in out and "policy_trainer/grad_norm" in out
    assert (tmp_path / "out" / "metrics.jsonl").exists()
