"""Configuration dataclasses (same field names and defaults as the reference's
``chatlearn/configs``) and the YAML/dot-list resolver that instantiates them."""
from .base import BaseConfig, BaseModelConfig, FreeGpuMemoryConfig
from .common import (OptimizerConfig, PartialRolloutManagerConfig, PolicyTrainerConfig,
                     RefPolicyConfig, RewardConfig, RolloutManagerConfig)
from .conf import (MISSING, ConfigError, apply_dotlist, load_yaml, merge, missing_keys, resolve,
                   to_container, to_dataclass)
from .fsdp_config import FSDPConfig, FSDPPolicyTrainerConfig, FSDPRefPolicyConfig
from .megatron_config import (MegatronConfig, MegatronModelArchitectureConfig,
                              MegatronPolicyTrainerConfig, MegatronRefPolicyConfig)
from .policy_config import PolicyConfig, RolloutConfig
from .runtime_config import LogConfig, RuntimeConfig, RuntimeEnvConfig
