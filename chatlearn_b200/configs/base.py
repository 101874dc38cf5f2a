"""Config base classes.

Parity: chatlearn/configs/base/base_config.py:5-70 (dict-like dataclass whose
``validate()`` / ``__post_init__`` walk the MRO and call every class's
``_validate_impl`` / ``_post_init_impl``) and
chatlearn/configs/base/base_model_config.py:7-94 (fields common to all models).
"""
from dataclasses import dataclass, field, fields, is_dataclass
from typing import Any, Dict, Optional

from .conf import MISSING  # noqa: F401  (re-exported)


@dataclass
class BaseConfig:
    """Dataclass with dict-style access and MRO-wide validation hooks."""

    def __getitem__(self, key):
        return getattr(self, key)

    def __setitem__(self, key, value):
        setattr(self, key, value)

    def __contains__(self, key):
        return hasattr(self, key)

    def get(self, key, default=None):
        return getattr(self, key, default)

    def keys(self):
        return [f.name for f in fields(self)]

    def items(self):
        return [(k, getattr(self, k)) for k in self.keys()]

    def _run_mro(self, method):
        seen = set()
        for klass in reversed(type(self).__mro__):
            fn = klass.__dict__.get(method)
            if fn is not None and fn not in seen:
                seen.add(fn)
                fn(self)

    def __post_init__(self):
        self._run_mro("_post_init_impl")

    def validate(self):
        """Run ``_validate_impl`` of every class in the MRO, then recurse."""
        self._run_mro("_validate_impl")
        for f in fields(self):
            v = getattr(self, f.name)
            if isinstance(v, BaseConfig):
                v.validate()
            elif isinstance(v, dict):
                for vv in v.values():
                    if isinstance(vv, BaseConfig):
                        vv.validate()

    def _post_init_impl(self):
        pass

    def _validate_impl(self):
        pass


@dataclass
class FreeGpuMemoryConfig(BaseConfig):
    offload_weights: bool = False
    free_grad_buffers: bool = False
    offload_optimizer_states: bool = False


@dataclass
class BaseModelConfig(BaseConfig):
    """Settings shared by every model role."""
    num_gpu: int = 0
    num_cpu: int = 0
    gpu_per_process: Optional[int] = None
    cpu_per_process: Optional[int] = None
    trainable: bool = False
    packing: bool = False
    max_token_in_packing: int = 32768
    generation_batch_size: int = 1
    sync_frequency: int = 1
    free_gpu_memory: FreeGpuMemoryConfig = field(default_factory=FreeGpuMemoryConfig)
    load: Optional[str] = None
    # HF-style architecture dict for random-init models (used when ``load`` has no
    # config.json, e.g. synthetic benchmarks); not present in the reference schema.
    model_arch: Optional[Dict[str, Any]] = None
    seed: int = 1234
    replica_dp_size: Optional[int] = None
    num_replica: int = 1
    trust_remote_code: bool = True
    num_inference_per_prompt: int = 32
    enable_thinking: bool = False
    max_prompt_tokens_length: int = 1024
    max_response_tokens_length: int = 2048

    def _validate_impl(self):
        assert self.num_gpu >= 0 and self.num_cpu >= 0
        assert not (self.num_gpu > 0 and self.num_cpu > 0), \
            "a model runs on GPUs or on CPUs, not both"
        if self.num_gpu > 0 and self.gpu_per_process is not None:
            assert self.gpu_per_process == 1, "one process per GPU"
        assert self.sync_frequency >= 1


def asdict_shallow(cfg):
    return {f.name: getattr(cfg, f.name) for f in fields(cfg)} if is_dataclass(cfg) else dict(cfg)
