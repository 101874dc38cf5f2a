"""chatlearn_b200 — a Blackwell-native RL post-training framework.

Public API (same names as ``chatlearn/__init__.py:19-32`` of the reference):
``init``, ``BaseModule``, ``TorchModule``, ``FSDPModule``, ``MegatronModule``,
``Engine``, ``RLHFEngine``, ``Environment``, ``Trainer``, ``Evaluator``,
``ControlDependencies``, ``get``, ``get_args``, ``logger``.
"""
__version__ = "0.1.0"

_LAZY = {
    "init": ("chatlearn_b200.launcher.initialize", "init"),
    "BaseModule": ("chatlearn_b200.models.base_module", "BaseModule"),
    "TorchModule": ("chatlearn_b200.models.base_module", "TorchModule"),
    "FSDPModule": ("chatlearn_b200.models.fsdp_module", "FSDPModule"),
    "MegatronModule": ("chatlearn_b200.models.megatron_module", "MegatronModule"),
    "RolloutModule": ("chatlearn_b200.models.rollout_module", "RolloutModule"),
    "Engine": ("chatlearn_b200.runtime.engine", "Engine"),
    "RLHFEngine": ("chatlearn_b200.runtime.engine", "RLHFEngine"),
    "Environment": ("chatlearn_b200.runtime.environment", "Environment"),
    "Trainer": ("chatlearn_b200.runtime.trainer", "Trainer"),
    "Evaluator": ("chatlearn_b200.runtime.evaluator", "Evaluator"),
    "ControlDependencies": ("chatlearn_b200.runtime.model_flow", "ControlDependencies"),
    "get": ("chatlearn_b200.utils.future", "get"),
    "get_args": ("chatlearn_b200.utils.global_vars", "get_args"),
    "logger": ("chatlearn_b200.utils.logger", "logger"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(f"module 'chatlearn_b200' has no attribute '{name}'")
