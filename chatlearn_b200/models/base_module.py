"""Worker base classes: lifecycle, data loading, metrics, residency hooks.

Parity: chatlearn/models/base_module.py:45-728 and
chatlearn/models/torch_module.py:40-194.  In the reference every module instance
is a Ray actor pinned to a (fraction of a) GPU and the driver calls its methods
remotely.  Here the job is SPMD — one process per GPU, every role instantiated
in every process — so a module carries its *placement* (the global ranks that
host it) and the engine calls the same methods locally on those ranks.  The
method surface a user overrides (``setup``, ``forward_step``, ``train_step``,
``eval_forward``, ``save_checkpoint``, ``onload``/``offload``, metrics) is the
reference's.
"""
import os
import time
from itertools import cycle
from typing import Any, Dict, List

import torch

from chatlearn_b200.data.data import RLHFDataLoader
from chatlearn_b200.data.sampler import MultiDatasetSampler
from chatlearn_b200.utils.global_vars import get_args, set_global_variables
from chatlearn_b200.utils.logger import model_logger
from chatlearn_b200.utils.timer import Timers
from chatlearn_b200.utils.utils import map_reduce_metrics


class BaseModule:
    """Base of every role (policy, trainer, reference, reward, managers)."""

    def __init__(self, name: str, args=None, replica_id: int = 0):
        self.name = name
        if args is not None:
            set_global_variables(args)
        self.global_args = get_args()
        margs = self.global_args.models[name]
        self._module_args = margs
        self._runtime_args = self.global_args.runtime_args
        self.total_gpu = margs.num_gpu
        self.total_cpu = margs.num_cpu
        self.trainable = margs.trainable
        self.replica_id = replica_id
        self._num_replica = max(int(getattr(margs, "num_replica", 1) or 1), 1)
        self._is_colocate = False
        # placement, filled by the scheduler
        self.placement: List[int] = []          # global ranks hosting this role
        self.role_rank: int = -1                # index of this process in ``placement``
        self.mesh = None                        # parallel.Mesh of the role
        # data
        self._dataloader = self._eval_dataloader = None
        self._data_iter = self._eval_data_iter = None
        self._all_datasets = self._all_eval_datasets = None
        # bookkeeping
        self._timers = Timers()
        self._iteration = 0
        self._train_iteration = 0
        self._episode_id = 0
        self._resume_training = False
        self._metric_prefix = name
        self._metric_list: List[Dict[str, Any]] = []
        self._peak_memory = 0.0
        self._logger = model_logger(name)
        self.call_funcs: List[str] = []
        self.trainable_funcs: List[str] = []
        self.error_signal = None
        self.profiler = None
        self._consumed_samples = int(self._runtime_args.consumed_samples or 0)

    # ------------------------------------------------------------------ identity
    @property
    def module_args(self):
        return self._module_args

    @property
    def runtime_args(self):
        return self._runtime_args

    def get_runtime_args(self):
        return self._runtime_args

    @property
    def is_colocate(self):
        return self._is_colocate

    def set_colocate(self, flag: bool):
        self._is_colocate = flag

    @property
    def num_replica(self) -> int:
        return self._num_replica

    @property
    def num_gpu_per_replica(self) -> int:
        return max(self.total_gpu // self._num_replica, 1) if self.total_gpu else 0

    @property
    def is_member(self) -> bool:
        """Whether this process hosts the role."""
        return self.role_rank >= 0

    @property
    def replica_index(self) -> int:
        """Replica this process belongs to (rollout: one engine per replica)."""
        if self.total_gpu == 0 or self.role_rank < 0:
            return max(self.role_rank, 0)
        return self.role_rank // self.num_gpu_per_replica

    @property
    def is_replica_leader(self) -> bool:
        if self.role_rank < 0:
            return False
        if self.total_gpu == 0:
            return True
        return self.role_rank % self.num_gpu_per_replica == 0

    @property
    def is_data_leader(self) -> bool:
        """Whether this rank publishes the outputs of its data-parallel rank (one
        rank per model-parallel group does)."""
        return self.is_replica_leader

    # data parallel view used by the executor to slice batches
    @property
    def data_parallel_size(self) -> int:
        if self.total_gpu == 0:
            return max(len(self.placement), 1)
        return self._num_replica * int(getattr(self._module_args, "replica_dp_size", 1) or 1)

    @property
    def data_parallel_rank(self) -> int:
        if self.role_rank < 0:
            return -1
        if self.total_gpu == 0:
            return self.role_rank
        if self.mesh is not None and self.mesh.coords:
            return self.replica_index * int(getattr(self._module_args, "replica_dp_size", 1) or 1) \
                + self.mesh.coords.get("dp_outer", 0)
        return self.replica_index

    def get_data_parallel_size(self):
        return self.data_parallel_size

    def get_data_parallel_rank(self):
        return self.data_parallel_rank

    def get_rank(self):
        return int(os.environ.get("RANK", "0"))

    def get_address(self):
        return os.environ.get("MASTER_ADDR", "127.0.0.1")

    def get_visible_gpus(self):
        return [int(os.environ.get("LOCAL_RANK", "0"))] if self.total_gpu else []

    def is_master_node(self):
        return self.get_rank() == 0

    # ------------------------------------------------------------------ lifecycle
    def init(self):
        """Distributed environment set-up of the role (process groups)."""

    def setup(self):
        """Create the model / optimizer / engine.  User hook."""

    def model_setup(self):
        """Called by the engine on every hosting rank after ``init``."""
        self.global_args.active_module_args = self._module_args
        if self._runtime_args.data_checkpoint_path and self._runtime_args.enable_resume_training:
            from chatlearn_b200.checkpoint.checkpoint_manager import CheckpointManager
            self._data_ckpt_manager = CheckpointManager(
                self, self._runtime_args.data_checkpoint_path, self._runtime_args.max_data_ckpt_nums,
                self._runtime_args.load_data_checkpoint_iteration)
            meta = self._data_ckpt_manager.resume()
            if meta:
                self._resume_training = True
                self._consumed_samples = meta.get("consumed_samples", self._consumed_samples)
        self.setup()

    def validate(self):
        return "ok"

    def before_episode(self):
        pass

    def after_episode(self):
        pass

    def terminate(self):
        pass

    def train(self):
        pass

    def eval(self):
        pass

    def set_start_iteration(self, it: int):
        self._train_iteration = it

    # ------------------------------------------------------------------ compute hooks
    def forward_step(self, data: List[Dict], iteration: int = 0, **kwargs) -> List[Dict]:
        raise NotImplementedError

    def eval_forward(self, data: List[Dict], iteration: int = 0, **kwargs) -> List[Dict]:
        return self.forward_step(data, iteration, is_eval=True, **kwargs)

    def train_step(self, data_list: List[Dict], **kwargs):
        raise NotImplementedError

    def save_checkpoint(self, iteration: int):
        pass

    def save_data_checkpoint(self, replica_id: int, iteration: int, episode_id: int):
        mgr = getattr(self, "_data_ckpt_manager", None)
        if mgr is not None:
            self._consumed_samples = self._runtime_args.consumed_samples
            mgr.save_checkpoint(replica_id, iteration, episode_id, self._consumed_samples)

    # ------------------------------------------------------------------ data
    def build_dataset(self, prompts: List[Dict], is_eval: bool = False):
        """Override to customise: raw records → indexable dataset."""
        from chatlearn_b200.data.prompt_dataset import PromptPipeline, VLPromptPipeline
        from chatlearn_b200.data.tokenizer import load_tokenizer
        tok = getattr(self, "tokenizer", None)
        if tok is None:
            needs_tok = any(p.get("input_ids") is None for p in prompts[:8])
            if needs_tok:
                tok = load_tokenizer(getattr(self._module_args, "load", None))
                self.tokenizer = tok
        max_len = int(getattr(self._module_args, "max_prompt_tokens_length", 1 << 30))
        think = getattr(self._module_args, "enable_thinking", False)
        if self._runtime_args.model_type == "vlm":
            arch = getattr(self, "arch", None)
            vc = (getattr(arch, "vision_config", None) or {}) if arch is not None else {}
            return VLPromptPipeline(prompts, max_len, tok, enable_thinking=think, raw_chat=self._runtime_args.raw_chat,
                                    image_token_id=getattr(arch, "image_token_id", None),
                                    video_token_id=getattr(arch, "video_token_id", None),
                                    tokens_per_second=float(vc.get("tokens_per_second", 1)),
                                    merge_size=int(vc.get("spatial_merge_size", 2)),
                                    patch_size=int(vc.get("patch_size", 14)),
                                    temporal_patch_size=int(vc.get("temporal_patch_size", 2)),
                                    # Qwen3-VL normalises to [-1, 1]; Qwen2.5-VL uses the CLIP statistics
                                    mean=(0.5, 0.5, 0.5) if "num_position_embeddings" in vc else None,
                                    std=(0.5, 0.5, 0.5) if "num_position_embeddings" in vc else None,
                                    max_pixels=int(getattr(self._module_args, "max_pixels", 14 * 14 * 4 * 1280)))
        return PromptPipeline(prompts, max_len, tok, enable_thinking=think, raw_chat=self._runtime_args.raw_chat)

    @property
    def loader_parallel_size(self) -> int:
        """Number of ways the prompt stream is split (``replica_index`` is this process's part)."""
        return self.num_replica

    def build_all_dataset(self, prompts_list: List[List[Dict]], is_eval: bool = False):
        return [self.build_dataset(p, is_eval) for p in prompts_list]

    def _build_dataloader(self, data: List[List[Dict]], sample_per_episode: int, is_eval: bool = False):
        datasets = self.build_all_dataset(data, is_eval)
        n = 1 if is_eval else int(self._runtime_args.num_inference_per_prompt)
        sampler = MultiDatasetSampler(
            dataset_sizes=[len(d) for d in datasets], sample_per_episode=sample_per_episode,
            data_ratio=self._runtime_args.data_ratio, consumed_samples=self._consumed_samples,
            num_inference_per_prompt=n, shuffle=self._runtime_args.data_shuffle and not is_eval,
            is_eval=is_eval, data_parallel_rank=self.replica_index,
            data_parallel_size=self.loader_parallel_size, drop_last="cycle",
            data_rerank=self._runtime_args.data_rerank, seed=int(getattr(self._module_args, "seed", 0)))
        loader = RLHFDataLoader(datasets, sampler, data_parallel_rank=self.replica_index,
                                data_parallel_size=self.loader_parallel_size, num_inference_per_prompt=n)
        if is_eval:
            self._eval_dataloader, self._eval_data_iter = loader, iter(loader)
            self._all_eval_datasets = datasets
        else:
            self._dataloader, self._data_iter = loader, iter(loader)
            self._all_datasets = datasets
        return loader

    def reset_eval_data_iter(self):
        if self._eval_dataloader is not None:
            self._eval_data_iter = iter(self._eval_dataloader)

    def next_batch(self, is_eval: bool = False) -> List[Dict]:
        """This replica's samples of the next episode."""
        it = self._eval_data_iter if is_eval else self._data_iter
        return next(it)

    # ------------------------------------------------------------------ metrics / timers
    def timers(self, name):
        return self._timers(name)

    def timer_summary(self, e2e_cost=None):
        return self._timers.log(return_dict=True)

    def get_and_clear_metrics(self):
        if not self._metric_list:
            return self._metric_prefix, {}
        m = map_reduce_metrics(self._metric_list)
        self._metric_list = []
        return self._metric_prefix, m

    def peak_memory(self) -> float:
        return self._peak_memory

    # ------------------------------------------------------------------ residency
    def onload(self, **kwargs):
        pass

    def offload(self, **kwargs):
        pass

    def empty_cache(self):
        pass

    # ------------------------------------------------------------------ parameter sync hooks
    def get_parameter_layout(self):
        """``{leaf name: (tensor, Leaf)}`` of this rank, see synchronizer."""
        return {}

    def pre_parameter_sync(self):
        pass

    def post_parameter_sync(self):
        pass

    def get_gpu_info(self):
        if torch.cuda.is_available():
            return int(os.environ.get("LOCAL_RANK", "0")), torch.cuda.get_device_name()
        return -1, "cpu"

    def get_mem_info(self):
        if torch.cuda.is_available():
            return torch.cuda.mem_get_info()
        return (0, 0)

    # ------------------------------------------------------------------ stage resume
    def enable_stage_resume(self, is_eval: bool) -> bool:
        return (not is_eval and bool(getattr(self._module_args, "enable_stage_resume", False))
                and bool(self._runtime_args.data_checkpoint_path))

    def get_stage_outputs_path(self, iteration: int) -> str:
        return os.path.join(self._runtime_args.data_checkpoint_path, str(iteration),
                            f"{self.name}_replica_{self.replica_index}.pt")

    def load_stage_outputs(self, is_eval: bool, iteration: int):
        if not self.enable_stage_resume(is_eval):
            return None
        path = self.get_stage_outputs_path(iteration)
        if os.path.exists(path):
            return torch.load(path, weights_only=False)
        return None

    def save_stage_outputs(self, is_eval: bool, outputs, iteration: int):
        if not self.enable_stage_resume(is_eval) or not self.is_replica_leader:
            return
        path = self.get_stage_outputs_path(iteration)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        torch.save(outputs, path)


class TorchModule(BaseModule):
    """Module with a torch model on a device: device selection, profiler, memory
    statistics and the tagged onload/offload order with barriers."""

    def __init__(self, name: str, args=None, replica_id: int = 0):
        super().__init__(name, args, replica_id)
        self.device = torch.device("cpu")
        self._residency = None
        self._resident = {"weights": True, "optimizer": True, "grads": True}

    def model_setup(self):
        if self.total_gpu > 0 and torch.cuda.is_available():
            self.device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
            torch.cuda.set_device(self.device)
        super().model_setup()
        if self._runtime_args.profiler_dir and self.replica_index == 0:
            self._setup_profiler()

    def _setup_profiler(self):
        acts = [torch.profiler.ProfilerActivity.CPU]
        if self.device.type == "cuda":
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        out = os.path.join(self._runtime_args.profiler_dir, f"{self.name}_rank{self.get_rank()}")
        self.profiler = torch.profiler.profile(
            activities=acts, schedule=torch.profiler.schedule(wait=1, warmup=1, active=1),
            on_trace_ready=torch.profiler.tensorboard_trace_handler(out), record_shapes=False)

    @property
    def group(self):
        """Process group wrapper spanning the role (barriers of onload/offload)."""
        return self.mesh.groups.get("world") if self.mesh is not None else None

    def _barrier(self):
        g = getattr(self, "role_group", None)
        if g is not None and g.size > 1:
            g.barrier()

    def peak_memory(self):
        if self.device.type == "cuda":
            self._peak_memory = max(self._peak_memory,
                                    torch.cuda.max_memory_allocated(self.device) / (1 << 30))
        return self._peak_memory

    def empty_cache(self):
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    # subclasses provide the tagged tensor sets
    def _tagged(self, tag: str):
        return []

    def _release(self, owner, attr):
        setattr(owner, attr, None)

    def _rebind(self, owner, attr, tensor):
        setattr(owner, attr, tensor)

    def _residency_mgr(self):
        if self._residency is None:
            from chatlearn_b200.utils.flat_tensors import ResidencyManager
            self._residency = ResidencyManager(self.device)
        return self._residency

    def offload(self, to_offload_weights=None, to_free_grad_buffers=None,
                to_offload_optimizer_states=None, **kwargs):
        """Release device memory by tag according to ``free_gpu_memory`` (or the
        explicit arguments); order and barriers follow torch_module.py:123-194."""
        if not self.is_member:
            return
        fg = self._module_args.free_gpu_memory
        w = fg.offload_weights if to_offload_weights is None else to_offload_weights
        g = fg.free_grad_buffers if to_free_grad_buffers is None else to_free_grad_buffers
        o = fg.offload_optimizer_states if to_offload_optimizer_states is None else to_offload_optimizer_states
        if not (w or g or o):
            return
        self._barrier()
        t0 = time.perf_counter()
        mgr = self._residency_mgr()
        for tag, on in (("weights", w), ("optimizer", o), ("grads", g)):
            if on and self._resident.get(tag, False):
                if tag == "grads":
                    for owner, attr in self._tagged(tag):
                        self._release(owner, attr)
                elif tag == "weights" and self._weights_regenerable():
                    # the resident fp32 master shards contain the weights: drop the compute copy
                    # instead of moving it to the host, rebuild it by a cast when it is needed again
                    for owner, attr in self._tagged(tag):
                        self._release(owner, attr)
                    self._weights_dropped = True
                else:
                    # a frozen model's weights never change: after the first offload the
                    # host copy stays valid and later offloads only drop the device copy
                    mgr.offload(self._tagged(tag), self._release,
                                unchanged=(tag == "weights" and not self.trainable))
                self._resident[tag] = False
        self._barrier()
        self.empty_cache()
        self._metric_list.append({"offload_s": time.perf_counter() - t0})
        if self.device.type == "cuda":
            self._logger.debug(f"offload(w={w}, o={o}, g={g}) -> {torch.cuda.memory_allocated() / 2**30:.1f} GiB allocated")

    def onload(self, to_onload_weights=None, to_build_grad_buffers=None,
               to_onload_optimizer_states=None, **kwargs):
        if not self.is_member:
            return
        fg = self._module_args.free_gpu_memory
        w = fg.offload_weights if to_onload_weights is None else to_onload_weights
        g = fg.free_grad_buffers if to_build_grad_buffers is None else to_build_grad_buffers
        o = fg.offload_optimizer_states if to_onload_optimizer_states is None else to_onload_optimizer_states
        if not (w or g or o):
            return
        self._barrier()
        t0 = time.perf_counter()
        mgr = self._residency_mgr()
        for tag, on in (("weights", w), ("grads", g), ("optimizer", o)):
            if on and not self._resident.get(tag, True):
                if tag == "grads":
                    self._build_grad_buffers()
                elif tag == "weights" and getattr(self, "_weights_dropped", False):
                    self._regenerate_weights()
                    self._weights_dropped = False
                else:
                    mgr.onload(self._tagged(tag), self._rebind)
                self._resident[tag] = True
        self._barrier()
        self._metric_list.append({"onload_s": time.perf_counter() - t0})

    def _build_grad_buffers(self):
        pass

    def _weights_regenerable(self) -> bool:
        """Whether the compute-dtype weights can be rebuilt on the device from other resident state."""
        return False

    def _regenerate_weights(self):
        raise NotImplementedError
