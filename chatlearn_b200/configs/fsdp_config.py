"""FSDP-style (ZeRO-3) trainer configuration.

Parity: chatlearn/configs/fsdp_config.py:10-52.
"""
from typing import Any
from dataclasses import dataclass

from .base import BaseConfig, BaseModelConfig
from .common import PolicyTrainerConfig, RefPolicyConfig


@dataclass
class FSDPConfig(BaseConfig):
    fsdp_size: int = 1
    ulysses_sequence_parallel_size: int = 1
    meta_init: bool = False
    # optimizer-step reduce-scatter / all-gather by this package's peer-memory kernels (GPU, 2..8 ranks)
    fused_optimizer_comm: bool = True
    # shard the compute-dtype parameters and the gradient accumulator as well (what the reference's
    # fully_shard(..., reshard_after_forward=True) does): 1/dp of everything resident, blocks gathered per
    # segment.  Off: parameters stay whole on every rank (fits dense models up to ~10B on 180 GB) and the
    # only parameter collectives are one reduce-scatter and one all-gather per optimizer step.
    reshard_after_forward: bool = False
    groupgemm: bool = False
    use_expandable_segments: bool = False

    def _post_init_impl(self):
        if isinstance(self, BaseModelConfig) and self.num_gpu:
            if self.fsdp_size in (-1, 0):
                self.fsdp_size = self.num_gpu
            sp = self.ulysses_sequence_parallel_size
            denom = sp * max(self.num_replica, 1)
            if self.num_gpu % denom == 0:
                self.replica_dp_size = self.num_gpu // denom

    def _validate_impl(self):
        if isinstance(self, BaseModelConfig):
            assert self.num_gpu > 0, "the FSDP backend needs GPUs (or CPU ranks standing in for them)"
            sp = self.ulysses_sequence_parallel_size
            assert self.num_gpu % sp == 0, "num_gpu must be a multiple of ulysses_sequence_parallel_size"
            assert self.fsdp_size >= 1 and self.num_gpu % self.fsdp_size == 0, \
                "num_gpu must be a multiple of fsdp_size"
            assert self.fsdp_size % sp == 0, "fsdp_size must be a multiple of ulysses_sequence_parallel_size"


@dataclass
class FSDPRefPolicyConfig(RefPolicyConfig, FSDPConfig):
    pass


@dataclass
class FSDPPolicyTrainerConfig(PolicyTrainerConfig, FSDPConfig):
    gradient_checkpointing: bool = True
    # with gradient_checkpointing on: 'auto' keeps the activations of as many layers as the free
    # device memory holds and recomputes only the rest; an integer fixes the number recomputed
    checkpoint_layers: Any = "all"
    save_hf: bool = True
