"""The training engine: set-up, the episode loop, checkpoints, metrics.

Parity: chatlearn/runtime/engine.py:79-626 (``BaseEngine.setup``, ``Engine.learn``,
``logging_summary``, ``save_checkpoint``, ``_resume_from_data_checkpoint``,
``RLHFEngine``).  Episode structure is the reference's:

    sync parameters → [evaluate] → for each episode:
        make experiences → build the train stream (replay / advantages) →
        train → save checkpoint → sync parameters → evaluate → log

Every rank runs this loop (SPMD); phases are timed with CUDA events and the
summary reports the maximum over ranks.
"""
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from chatlearn_b200.data.data import StreamDataset
from chatlearn_b200.runtime.environment import Environment
from chatlearn_b200.runtime.evaluator import Evaluator
from chatlearn_b200.runtime.trainer import Trainer
from chatlearn_b200.schedule.metric_manager import MetricManager
from chatlearn_b200.schedule.model_manager import ModelManager
from chatlearn_b200.schedule.resource_manager import ResourceManager
from chatlearn_b200.utils.constant import LOG_START
from chatlearn_b200.utils.global_vars import get_args
from chatlearn_b200.utils.logger import logger
from chatlearn_b200.utils import trace
from chatlearn_b200.utils.timer import Timers


def _max_over_ranks(values: Dict[str, float]) -> Dict[str, float]:
    if not dist.is_initialized() or dist.get_world_size() == 1 or not values:
        return values
    keys = sorted(values)
    dev = "cuda" if (torch.cuda.is_available() and dist.get_backend() != "gloo") else "cpu"
    t = torch.tensor([values[k] for k in keys], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return dict(zip(keys, t.tolist()))


class BaseEngine:
    def __init__(self, models):
        self._models = list(models or [])
        self.global_args = get_args()
        self.runtime_args = self.global_args.runtime_args
        self.timers = Timers()
        self.model_manager: Optional[ModelManager] = None
        self.metric_manager: Optional[MetricManager] = None
        self._setup_done = False
        self.remote_models: List = []
        self.named_models: Dict[str, object] = {}

    def _create_remote_models(self):
        rm = ResourceManager(self._models)
        self.model_manager = ModelManager(self._models, rm, self.global_args)
        self.model_manager.create_dist_models()
        self.remote_models = self.model_manager.dist_models
        self.named_models = {m.name: m for m in self.remote_models}

    def setup(self):
        logger.info(f"{LOG_START} engine setup")
        self.timers("setup").start()
        self._create_remote_models()
        self.metric_manager = MetricManager(self.global_args)
        # process groups are created collectively, in model order, on every rank
        for m in self.remote_models:
            m.init()
        for m in self.remote_models:
            if m.is_member:
                self.timers(f"setup_{m.name}").start()
                m.model_setup()
                # colocated roles release what their config lets them release before the
                # next role is built (the reference offloads right after setup_engine /
                # model_setup, runtime/engine.py:103-130)
                if m.is_colocate:
                    m.offload()
                self.timers(f"setup_{m.name}").stop()
                if torch.cuda.is_available():
                    logger.debug(f"setup {m.name}: {torch.cuda.memory_allocated() / 2**30:.1f} GiB allocated")
        for m in self.remote_models:
            if m.is_member:
                m.validate()
        self.timers("setup").stop()
        self._setup_done = True

    def before_episode(self):
        for m in self.remote_models:
            if m.is_member:
                m.before_episode()

    def after_episode(self):
        for m in self.remote_models:
            if m.is_member:
                m.after_episode()

    @property
    def models(self):
        return self.remote_models

    def get_model(self, name):
        return self.named_models[name]

    def stop(self):
        if self.model_manager:
            self.model_manager.clean()
        if self.metric_manager:
            self.metric_manager.stop()


class Engine(BaseEngine):
    def __init__(self, environment: Optional[Environment] = None, trainer: Optional[Trainer] = None,
                 evaluator: Optional[Evaluator] = None, name: str = "alignment", models=None):
        if models is None:
            models = []
        super().__init__(models)
        self.env, self.trainer, self.evaluator = environment, trainer, evaluator
        for ex in (environment, trainer, evaluator):
            if ex is not None:
                ex.set_timers(self.timers)
                ex.global_args = self.global_args
        self._name = name
        self._start_episode = 0
        self._all_datasets = None
        self._replay_sample_manager = None
        self._data_loader: Optional[StreamDataset] = None
        self._param_sync_pairs = []
        self._post_process = None
        self.episode_stats: List[Dict[str, float]] = []

    # ------------------------------------------------------------------ configuration API
    def set_parameter_sync(self, src_model, dst_model):
        self._param_sync_pairs.append((src_model, dst_model))
        return self

    def set_dataset(self, dataset):
        self._all_datasets = dataset
        return self

    def set_replay_sample_manager(self, manager):
        self._replay_sample_manager = manager
        return self

    def set_trainer(self, trainer):
        self.trainer = trainer
        return self

    def set_environment(self, env):
        self.env = env
        return self

    def set_evaluator(self, evaluator):
        self.evaluator = evaluator
        return self

    # ------------------------------------------------------------------ set-up
    def _create_remote_models(self):
        rm = ResourceManager(self._models)
        self.model_manager = ModelManager(self._models, rm, self.global_args)
        for s, d in self._param_sync_pairs:
            self.model_manager.set_parameter_sync(s, d)
        self.model_manager.create_dist_models()
        self.remote_models = self.model_manager.dist_models
        self.named_models = {m.name: m for m in self.remote_models}

    def setup(self):
        super().setup()
        self._executors = [e for e in (self.env, self.trainer, self.evaluator) if e is not None]
        for ex in self._executors:
            ex.update_models(self.remote_models)
        if self.env is not None:
            self.env.set_multiple_datasets(self._all_datasets)
        self.timers("build_sync_parameter_groups").start()
        self.model_manager.build_parameter_group()
        self.timers("build_sync_parameter_groups").stop()
        for ex in self._executors:
            ex.setup()

    # ------------------------------------------------------------------ checkpoints
    def _resume_from_data_checkpoint(self):
        ra = self.runtime_args
        if not (ra.data_checkpoint_path and ra.enable_resume_training):
            return
        from chatlearn_b200.checkpoint.checkpoint_manager import CheckpointManager
        first = self.env.first_model() if self.env else None
        if first is None:
            return
        mgr = getattr(first, "_data_ckpt_manager", None) or CheckpointManager(
            first, ra.data_checkpoint_path, ra.max_data_ckpt_nums, ra.load_data_checkpoint_iteration)
        meta = mgr.resume()
        if meta:
            self._start_episode = meta["episode"] + 1
            ra.consumed_samples = meta["consumed_samples"]
            if self.trainer:
                self.trainer.set_start_iteration(meta["train_iteration"])
            logger.info(f"resume: start episode {self._start_episode}, consumed {ra.consumed_samples}")

    def save_checkpoint(self, episode_id: int):
        ra = self.runtime_args
        interval = ra.save_episode_interval
        if not interval or (episode_id + 1) % interval != 0 and episode_id + 1 != ra.num_episode:
            return
        self.timers("save_checkpoint").start()
        for m in self.remote_models:
            if m.trainable and m.is_member:
                m.onload(to_onload_weights=True, to_build_grad_buffers=False,
                         to_onload_optimizer_states=True)
                m.save_checkpoint(self.trainer.iteration if self.trainer else episode_id)
                if m.is_colocate:
                    m.offload()
        if ra.data_checkpoint_path and self.env is not None:
            first = self.env.first_model()
            if first.is_member and first.is_replica_leader:
                from chatlearn_b200.checkpoint.checkpoint_manager import CheckpointManager
                mgr = getattr(first, "_data_ckpt_manager", None)
                if mgr is None:
                    mgr = CheckpointManager(first, ra.data_checkpoint_path, ra.max_data_ckpt_nums)
                    first._data_ckpt_manager = mgr
                mgr.save_checkpoint(first.replica_index, self.trainer.iteration if self.trainer else 0,
                                    episode_id, int(ra.consumed_samples))
        self.timers("save_checkpoint").stop()

    # ------------------------------------------------------------------ evaluation / logging
    def evaluate(self, episode_id: int):
        ra = self.runtime_args
        if self.evaluator is None or not ra.eval_episode_interval:
            return
        if (episode_id + 1) % ra.eval_episode_interval != 0:
            return
        self.timers("evaluate").start()
        self.evaluator.eval(episode_id, self.trainer.iteration if self.trainer else 0)
        self.timers("evaluate").stop()

    def logging_summary(self, episode_id: int, episode_tokens: int = 0, num_samples: int = 0):
        names = ["episode", "environment", "train", "sync_parameters", "save_checkpoint", "evaluate"]
        local = self.timers.log(names, return_dict=True, reset=True)
        t = _max_over_ranks(local)
        summary = dict(t)
        ep = t.get("episode", 0.0)
        if ep > 0:
            summary["tps_throughput"] = episode_tokens / ep
            summary["samples_per_s"] = num_samples / ep
        step = self.trainer.iteration if self.trainer else episode_id
        self.metric_manager.log("engine/timer_summary", step, summary)
        # every role reports through its first rank; rank 0 writes the sinks
        mine = {}
        for m in self.remote_models:
            if not m.is_member:
                continue
            tm = m.timer_summary()
            prefix, metrics = m.get_and_clear_metrics()
            metrics = dict(metrics)
            for k, v in tm.items():
                metrics[f"{k}_total_s"] = v
            metrics["peak_memory_gib"] = m.peak_memory()
            if m.role_rank == 0:
                mine[prefix] = metrics
        from chatlearn_b200.runtime.executor import all_gather_objects
        for part in all_gather_objects(mine):
            for prefix, metrics in part.items():
                self.metric_manager.log(prefix, step, metrics)
        for ex in (self.env, self.trainer, self.evaluator):
            if ex is not None:
                prefix, metrics = ex.get_and_clear_metrics()
                self.metric_manager.log(prefix, step, metrics)
        if self._data_loader is not None:
            prefix, metrics = self._data_loader.get_and_clear_metrics()
            self.metric_manager.log(prefix, step, metrics)
        summary["episode_id"] = episode_id
        self.episode_stats.append(summary)
        return summary

    # ------------------------------------------------------------------ the loop
    def prepare(self):
        """Everything ``learn`` does before the first episode: set-up, resume, the
        train stream and the initial trainer -> rollout weight sync."""
        ra = self.runtime_args
        if not self._setup_done:
            self.setup()
        self._resume_from_data_checkpoint()
        n_mini = max(int(ra.sample_per_episode) // int(ra.train_global_batch_size), 1)
        self._data_loader = StreamDataset(
            ra.stream_data_loader_type, n_mini, self._replay_sample_manager,
            int(ra.train_micro_batch_size), ra.max_replay_episode, ra.replay_episode_offset)
        if self.trainer:
            self.trainer.set_data_loader(self._data_loader)
        dump = os.environ.get("DEBUG_SYNC_PARAMETERS_PATH")
        self.timers("sync_parameters").start()
        self.model_manager.sync_parameters(episode_offset=0)
        self.timers("sync_parameters").stop()
        if dump:
            # what the rollout holds after the sync, and what the trainer says it should hold;
            # `python -m chatlearn_b200.synchronizer.check_parameter_sync --root_dir <dump>` compares them
            from chatlearn_b200.synchronizer.check_parameter_sync import dump_expected
            for src, dst in self._param_sync_pairs:
                if dst.is_member and hasattr(dst, "dump_parameters"):
                    dst.dump_parameters(os.path.join(dump, "after_sync_parameter"))
                dump_expected(src, os.path.join(dump, "trainer_hf"))
        if ra.enable_eval_before_training and self.evaluator is not None:
            self.evaluator.eval(-1, 0)
        self._prepared = True

    def run_episode(self, episode_id: int):
        """One episode: rollout + scoring + reward → train → checkpoint → weight sync
        → evaluation → summary.  Returns the episode summary dict."""
        ra = self.runtime_args
        if ra.nsys and torch.cuda.is_available():
            if episode_id == ra.profile_episode:
                torch.cuda.cudart().cudaProfilerStart()
            elif episode_id == ra.profile_episode + 1:
                torch.cuda.cudart().cudaProfilerStop()
        self.timers("episode").start()
        self.before_episode()
        logger.info(f"{LOG_START} episode {episode_id} start")
        self.timers("environment").start()
        if os.environ.get("SKIP_GENERATION") is None:
            with trace.span("environment"):
                samples = self.env.make_experiences(episode_id)
        else:
            samples = []
        self.timers("environment").stop()
        with trace.span("replay_buffer"):
            self._data_loader.set_dataset([samples], episode_id, int(ra.sample_per_episode))
            tokens = self._data_loader.get_total_train_tokens()
            n_samples = self._data_loader.total_samples()
        if self.trainer is not None and n_samples > 0:
            self.timers("train").start()
            with trace.span("train"):
                self.trainer.train(episode_id)
            self.timers("train").stop()
        with trace.span("save_checkpoint"):
            self.save_checkpoint(episode_id)
        self.timers("sync_parameters").start()
        with trace.span("sync_parameters"):
            self.model_manager.sync_parameters(episode_offset=episode_id + 1)
        self.timers("sync_parameters").stop()
        with trace.span("evaluate"):
            self.evaluate(episode_id)
        self.after_episode()
        self.timers("episode").stop()
        if trace.enabled() and (not dist.is_initialized() or dist.get_rank() == 0):
            trace.dump(logger.info)
        return self.logging_summary(episode_id, tokens, n_samples)

    def learn(self):
        ra = self.runtime_args
        self.timers("chatlearn").start()
        if not getattr(self, "_prepared", False):
            self.prepare()
        for episode_id in range(self._start_episode, int(ra.num_episode)):
            self.run_episode(episode_id)
        self.timers("chatlearn").stop()
        logger.info(f"{LOG_START} {self._name} finished in {self.timers('chatlearn').elapsed():.1f} s")
        return self.episode_stats


class RLHFEngine(Engine):
    """PPO-style RLHF: policy, reference, reward and value inference + policy and
    value trainers (chatlearn/runtime/engine.py:601-626)."""

    def __init__(self, policy, reference, reward, value, policy_trainer, value_trainer):
        def env_compute_flow(batch):
            policy_out = policy.forward_step(batch)
            ref_out = reference.forward_step(policy_out)
            value_out = value.forward_step(policy_out)
            reward_out = reward.forward_step(policy_out, ref_out, value_out)
            return value_out, reward_out

        def trainer_compute_flow(batch):
            policy_trainer.train_step(batch)
            value_trainer.train_step(batch)

        env = Environment(env_compute_flow)
        trainer = Trainer(trainer_compute_flow)
        super().__init__(env, trainer, name="rlhf",
                         models=[policy, reference, reward, value, policy_trainer, value_trainer])
        self.set_parameter_sync(policy_trainer, policy)
        self.set_parameter_sync(value_trainer, value)
