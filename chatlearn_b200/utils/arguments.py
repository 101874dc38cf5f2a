"""Legacy YAML configuration (``chatlearn.init()`` without arguments).

Parity: chatlearn/utils/arguments.py:46-121,350-539: a plain YAML file with
``runtime`` / ``runtime_env`` / ``models`` sections, ``${ENV_NAME:default}``
substitution, ``includes:`` merging and per-model ``model_config_file``.  Parsed
into the same dataclasses the Hydra-style path uses, so old config files keep
working with the new engine.
"""
import argparse
import os
import sys
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

from chatlearn_b200.configs import (BaseConfig, BaseModelConfig, RuntimeConfig, RuntimeEnvConfig, apply_dotlist,
                                    load_yaml, merge, resolve, to_dataclass)


@dataclass
class Config(BaseConfig):
    env_args: RuntimeEnvConfig = field(default_factory=RuntimeEnvConfig)
    runtime_args: RuntimeConfig = field(default_factory=RuntimeConfig)
    models: Dict[str, Any] = field(default_factory=dict)

    def validate(self):
        self.runtime_args.validate()
        for m in self.models.values():
            if isinstance(m, BaseConfig):
                m.validate()


def _model_cfg(d: Dict[str, Any], base_dir: str) -> BaseModelConfig:
    d = dict(d)
    mcf = d.pop("model_config_file", None)
    if mcf:
        path = mcf if os.path.isabs(mcf) else os.path.join(base_dir, mcf)
        d = merge(load_yaml(path), d)
    if "free_memory" in d:                       # legacy switch: one flag for everything
        on = bool(d.pop("free_memory"))
        d.setdefault("free_gpu_memory", {"offload_weights": on, "free_grad_buffers": on,
                                         "offload_optimizer_states": on})
    return to_dataclass(BaseModelConfig, d)


def parse_args(config_file: Optional[str] = None, overrides=None) -> Config:
    if config_file is None:
        ap = argparse.ArgumentParser(add_help=False)
        ap.add_argument("-c", "--config", default=os.environ.get("CHATLEARN_CONFIG"))
        ns, rest = ap.parse_known_args(sys.argv[1:])
        config_file = ns.config
        overrides = overrides or [r for r in rest if "=" in r]
    assert config_file, "no config file: pass -c <yaml> or set CHATLEARN_CONFIG"
    data = resolve(apply_dotlist(load_yaml(config_file), overrides or []))
    base = os.path.dirname(os.path.abspath(config_file))
    runtime = data.get("runtime_args", data.get("runtime", {})) or {}
    runtime.setdefault("train_backend", "fsdp")
    for k, v in (("output_dir", "./output"), ("data_path", ""), ("num_episode", 1), ("sample_per_episode", 1),
                 ("train_micro_batch_size", 1), ("train_global_batch_size", 1), ("save_episode_interval", 0)):
        runtime.setdefault(k, v)
    runtime.setdefault("log_args_dict", {"log_dir": runtime["output_dir"]})
    cfg = Config(env_args=to_dataclass(RuntimeEnvConfig, data.get("env_args", data.get("runtime_env", {}))),
                 runtime_args=to_dataclass(RuntimeConfig, runtime),
                 models={k: _model_cfg(v, base) for k, v in (data.get("models") or {}).items()})
    return cfg
