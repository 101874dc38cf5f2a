"""Rollout (policy inference) configuration.

Parity: chatlearn/configs/policy_config.py:6-103.  The reference asserts
EP == 1 and PP == 1 for rollout because vLLM's EP weight sync is unsupported
(policy_config.py:89); the native rollout engine supports TP and EP, so only
PP is rejected.
"""
from dataclasses import dataclass

from .base import BaseModelConfig


@dataclass
class RolloutConfig(BaseModelConfig):
    is_sync_mode: bool = True
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    # sampling
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    eval_temperature: float = 0.6
    eval_top_p: float = 0.95
    eval_top_k: int = 20
    eval_presence_penalty: float = 0.0
    eval_frequency_penalty: float = 0.0
    eval_repetition_penalty: float = 1.0
    vllm_prompt_key: str = "prompt"
    vllm_input_ids_key: str = "input_ids"
    # engine
    max_num_batched_tokens: int = 32768
    max_seq_len_to_capture: int = 2348
    gpu_memory_utilization: float = 0.8
    enforce_eager: bool = False
    kv_block_size: int = 64
    max_num_seqs: int = 256
    # agent tasks: "continuous" = every model turn is its own request in an open engine session (a trajectory's
    # next turn joins the running batch as soon as its tools return); "lockstep" = one batched call per round
    agent_scheduling: str = "continuous"


@dataclass
class PolicyConfig(RolloutConfig):
    seq_length: int = 2048
    enable_thinking: bool = False
    enable_stage_resume: bool = False

    def _post_init_impl(self):
        mp = (self.tensor_model_parallel_size * self.expert_model_parallel_size
              * self.pipeline_model_parallel_size)
        if self.num_gpu and self.num_gpu % mp == 0:
            self.num_replica = self.num_gpu // mp
            self.replica_dp_size = 1
        self.seq_length = self.max_prompt_tokens_length + self.max_response_tokens_length

    def _validate_impl(self):
        assert self.pipeline_model_parallel_size == 1, "rollout does not use pipeline parallelism"
        mp = self.tensor_model_parallel_size * self.expert_model_parallel_size
        assert self.num_gpu > 0 and self.num_gpu % mp == 0, \
            f"policy.num_gpu={self.num_gpu} must be a multiple of tp*ep={mp}"
        assert 0.0 < self.gpu_memory_utilization <= 1.0
