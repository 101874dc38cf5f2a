"""Role-level common configs.

Parity: chatlearn/configs/base/common.py:7-76 and
chatlearn/configs/partial_rollout_manager_config.py:7-28.
"""
from dataclasses import dataclass, field
from typing import List

from .base import BaseConfig, BaseModelConfig


@dataclass
class OptimizerConfig(BaseConfig):
    clip_grad: float = 1.0
    lr: float = 2e-6
    min_lr: float = 0.0
    weight_decay: float = 0.01
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8


@dataclass
class RefPolicyConfig(BaseModelConfig):
    """Frozen reference policy (KL anchor)."""


@dataclass
class RewardConfig(BaseModelConfig):
    """Rule reward (CPU role) or reward model."""


@dataclass
class RolloutManagerConfig(BaseModelConfig):
    use_dynamic_load_blance: bool = True  # spelling kept: it is a YAML key users already have
    max_concurrent_per_engine: int = 192


@dataclass
class PolicyTrainerConfig(BaseModelConfig):
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    entropy_coef: float = 0.0
    kl_coef: float = 0.0
    pos_clip_ratio: float = 0.2
    neg_clip_ratio: float = 0.2
    diff_clip_ratio: float = 10.0
    final_clip_ratio: float = 3.0
    use_group_sequence_policy: bool = False
    train_micro_batch_size: int = 1
    train_vision_tower: bool = False      # vision-language models: update the vision tower too (frozen otherwise)

    def _validate_impl(self):
        assert self.pos_clip_ratio >= 0 and self.neg_clip_ratio >= 0


@dataclass
class PartialRolloutManagerConfig(BaseModelConfig):
    max_rollout_round: int = 2
    mini_response_per_prompt: int = 16
    rollout_ratio: List[float] = field(default_factory=lambda: [0.5, 0.5])

    def _validate_impl(self):
        assert len(self.rollout_ratio) == self.max_rollout_round, \
            "rollout_ratio needs one entry per rollout round"
        assert abs(sum(self.rollout_ratio) - 1.0) < 1e-6, "rollout_ratio must sum to 1"
