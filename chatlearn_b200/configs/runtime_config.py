"""Runtime (engine-level) configuration.

Parity: chatlearn/configs/runtime_config.py:13-242 (``LogConfig``,
``RuntimeConfig``, ``RuntimeEnvConfig``).  Field names and defaults match so
reference YAML files load unchanged; fields that only configured Ray are kept
as inert values.
"""
from dataclasses import dataclass, field
from typing import List, Optional

from .base import BaseConfig
from .conf import MISSING


@dataclass
class LogConfig(BaseConfig):
    log_dir: str = MISSING
    enable_tensorboard: bool = False
    tensorboard_dir: Optional[str] = None
    enable_wandb: bool = False
    wandb_dir: Optional[str] = None
    wandb_project: Optional[str] = None
    wandb_id: Optional[str] = None
    wandb_name: Optional[str] = None
    wandb_resume: str = "allow"


@dataclass
class RuntimeConfig(BaseConfig):
    # setup
    train_backend: str = MISSING
    rollout_backend: str = "native"
    task_type: str = "chat"
    use_rollout_manager: bool = False
    use_partial_rollout: bool = False
    exp_name: str = "CHATLEARN"
    colocation: List[str] = field(default_factory=list)
    concurrent_setup: bool = False
    debug: bool = False
    nsys: bool = False
    # paths
    output_dir: str = MISSING
    profiler_dir: Optional[str] = None
    data_path: str = MISSING
    eval_data_path: Optional[str] = None
    data_checkpoint_path: Optional[str] = None
    # training
    num_episode: int = MISSING
    sample_per_episode: int = MISSING
    num_training_epoch: int = 1
    train_micro_batch_size: int = MISSING
    train_global_batch_size: int = MISSING
    num_inference_per_prompt: int = 32
    save_episode_interval: int = MISSING
    enable_resume_training: bool = True
    # data
    raw_chat: bool = False
    data_ratio: List[int] = field(default_factory=list)
    data_shuffle: bool = True
    data_rerank: bool = True
    max_replay_episode: int = 0
    replay_episode_offset: int = 0
    consumed_samples: int = 0
    max_data_ckpt_nums: Optional[int] = None
    load_data_checkpoint_iteration: Optional[int] = None
    stream_data_loader_type: str = "fixed"
    model_type: str = "llm"
    # eval
    eval_episode_interval: int = 0
    enable_eval_before_training: bool = False
    # memory / scheduling
    bucket_size_mb_in_memory_manager: float = 1024      # largest message of the point-to-point weight sync (MB)
    cpu_schedule_strategy: str = "SPREAD"
    policy_to_regroup_queue: str = "global_barrier"
    log_args_dict: LogConfig = field(default_factory=LogConfig)
    # profiling: episode at which the CUDA profiler range opens (the reference
    # hard-codes episode 4, runtime/engine.py:490-494)
    profile_episode: int = 4
    # liveness: seconds without a heartbeat before a rank is declared dead
    heartbeat_timeout_s: float = 60.0

    def _validate_impl(self):
        from chatlearn_b200.utils.constant import ROLLOUT_BACKENDS, TRAIN_BACKENDS
        if self.train_backend is not MISSING:
            assert self.train_backend in TRAIN_BACKENDS, \
                f"train_backend must be one of {TRAIN_BACKENDS}, got {self.train_backend}"
        assert self.rollout_backend in ROLLOUT_BACKENDS, \
            f"rollout_backend must be one of {ROLLOUT_BACKENDS}"
        assert self.stream_data_loader_type in ("fixed", "dynamic")
        assert self.model_type in ("llm", "vlm")
        assert self.task_type in ("chat", "agent")


@dataclass
class RuntimeEnvConfig(BaseConfig):
    """Launcher environment.  ``platform`` selects how ranks are spawned:
    ``local`` (this launcher forks one process per GPU) or ``torchrun`` (ranks
    already exist; read RANK/WORLD_SIZE from the environment)."""
    excludes: List[str] = field(default_factory=lambda: ["*pt", "logs", "tensorboards", ".nfs*"])
    platform: str = "local"
    pip: List[str] = field(default_factory=list)
    working_dir: Optional[str] = None
    py_modules: List[str] = field(default_factory=list)
