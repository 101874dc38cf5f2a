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


def test_megatron_architecture_block_is_filled_from_the_model_description():
    """Hybrid layer pattern, partial rotary, multimodal rotary sections and the YaRN factor reach the
    Megatron-style architecture block that tools and users inspect."""
    import dataclasses
    from chatlearn_b200.configs.megatron_config import MegatronModelArchitectureConfig as C
    from chatlearn_b200.models.nn import PRESETS
    from chatlearn_b200.utils.megatron_utils import arch_to_megatron_cfg

    def blank():
        req = {f.name: 1 for f in dataclasses.fields(C)
               if f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING}
        return C(**req)
    nxt = arch_to_megatron_cfg(PRESETS["tiny_qwen3_next"](), blank())
    assert nxt.hybrid_override_pattern == "M-M-M-*-" and nxt.is_hybrid_model and nxt.rotary_percent == 0.25
    assert nxt.moe_shared_expert_intermediate_size == 64 and nxt.num_experts == 8
    vl = arch_to_megatron_cfg(PRESETS["tiny_qwen2_5_vl"](), blank())
    assert vl.position_embedding_type == "mrope" and vl.mrope_section == [4, 6, 6]
    ds = PRESETS["deepseek_v3_671b"]()
    ds.rope_scaling = {"type": "yarn", "factor": 40}
    mc = arch_to_megatron_cfg(ds, blank())
    assert mc.multi_latent_attention and mc.rotary_scaling_factor == 40.0 and mc.moe_router_num_groups == 8


@pytest.mark.parametrize("name", sorted(f for f in os.listdir(os.path.join(ROOT, "examples")) if f.startswith("train_")))
def test_example_scripts_compose_into_configurations(name):
    """Every ``key=value`` override of a launch script names a field the configuration schema has and takes a
    value of its type (shell variables replaced by stand-ins)."""
    import re
    text = open(os.path.join(ROOT, "examples", name)).read().replace("\\\n", " ")
    text = re.sub(r"\$\(\(.*?\)\)", "64", text)              # shell arithmetic (contains spaces)
    algo = re.search(r"launch (\w+) --config-file", text).group(1)
    tpl = re.search(r"template/(\S+)", text).group(1)
    ov = [w for w in text.split() if re.match(r"^(runtime_args|models)\.[\w.]+=", w)]
    subs = ((r"\$\{CHATLEARN\}", "/x"), (r"\$\{exp_name\}", "e"), (r"\$\{num_device\}", "8"), (r"\$\(\(.*?\)\)", "64"),
            (r"\$\{\w+(:-(\w+))?\}", r"\2"))
    for pat, rep in subs:
        ov = [re.sub(pat, rep, o) for o in ov]
    cfg = _cfg(algo, tpl, ov)
    assert cfg.runtime_args.exp_name == "e"
