"""The shipped YAML templates compose into valid configurations."""
import os

import pytest

from chatlearn_b200.entrypoint import compose_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg(algo, template, overrides):
    import importlib
    from chatlearn_b200.entrypoint import ALGO_REGISTRY
    mod, _, cfg_cls = ALGO_REGISTRY[algo]
    cls = getattr(importlib.import_module(mod), cfg_cls)
    return compose_config(cls, os.path.join(ROOT, "template", template), overrides)


def test_grpo_fsdp_template():
    cfg = _cfg("grpo", "grpo_fsdp.yaml", ["runtime_args.output_dir=/tmp/o", "models.policy_trainer.num_gpu=4",
                                          "models.policy.tensor_model_parallel_size=2",
                                          "models.policy_trainer.model_arch={preset: qwen3_8b}"])
    cfg.validate()
    m = cfg.models
    assert m.ref_policy.num_gpu == 4 and m.policy.num_gpu == 4 and m.policy.num_replica == 2
    assert m.policy_trainer.trainable and m.policy_trainer.fsdp_size == 4
    assert cfg.runtime_args.data_checkpoint_path == "/tmp/o/data_checkpoint_path/"
    assert m.partial_rollout_manager.rollout_ratio == [0.5, 0.5]


def test_grpo_megatron_template():
    cfg = _cfg("grpo", "grpo_megatron.yaml", ["runtime_args.output_dir=/tmp/o"])
    cfg.validate()
    tr = cfg.models.policy_trainer
    assert tr.tensor_model_parallel_size == 2 and tr.expert_model_parallel_size == 4
    assert tr.seq_length == 1024 + 4096 and tr.megatron_model_cfg.num_experts == 128
    assert cfg.models.ref_policy.megatron_model_cfg.moe_router_topk == 8
    assert cfg.models.policy.expert_model_parallel_size == 8


def test_rlhf_template():
    cfg = _cfg("rlhf", "rlhf_fsdp.yaml", ["runtime_args.output_dir=/tmp/o"])
    cfg.validate()
    assert cfg.models.value_trainer is None and cfg.models.reward.clip_reward_value == 5.0
    assert cfg.runtime_args.init_kl_coef == 0.05


@pytest.mark.parametrize("name", sorted(f for f in os.listdir(os.path.join(ROOT, "examples")) if f.startswith("train_")))
def test_example_scripts_name_existing_templates(name):
    text = open(os.path.join(ROOT, "examples", name)).read()
    tpl = [w for w in text.split() if w.startswith("template/")]
    assert tpl and all(os.path.exists(os.path.join(ROOT, t)) for t in tpl)
