"""Rollout executor: one call = one episode of experience.

Parity: chatlearn/runtime/environment.py:83-158.  The first model of the flow
owns the prompt data loader (one per replica, sharded by replica id).
"""
from typing import Dict, List

from chatlearn_b200.runtime.executor import Executor
from chatlearn_b200.utils.logger import logger


class Environment(Executor):
    def __init__(self, model_flow):
        super().__init__(model_flow)
        self._all_datasets = None
        self.sample_per_episode = 0
        self._metric_prefix = "environment"
        self._episode = 0

    def set_multiple_datasets(self, all_datasets):
        self._all_datasets = all_datasets

    set_dataset = set_multiple_datasets

    def setup(self):
        super().setup()
        self.sample_per_episode = int(self.global_args.runtime_args.sample_per_episode)
        m = self.first_model()
        if m.is_member and self._all_datasets is not None:
            m._build_dataloader(self._all_datasets, self.sample_per_episode, is_eval=False)
            ds = m._all_datasets
            logger.info(f"{m.name}: {sum(len(d) for d in ds)} prompts in {len(ds)} dataset(s)")

    @property
    def global_dp_size(self) -> int:
        return self.first_model().data_parallel_size

    @property
    def batch_size(self) -> int:
        return int(self.first_model().module_args.generation_batch_size)

    def num_iteration(self) -> int:
        per_replica = self.sample_per_episode // max(self.global_dp_size, 1)
        bs = max(self.batch_size, 1)
        return (per_replica + bs - 1) // bs

    def make_experiences(self, episode: int = None) -> List[Dict]:
        ep = self._episode if episode is None else episode
        res = self.execute_flow(lambda model: model.next_batch(is_eval=False), ep, is_eval=False)
        self._episode = ep + 1
        nodes = list(res)
        merged = res[nodes[0]]
        for n in nodes[1:]:
            merged = [{**a, **b} for a, b in zip(merged, res[n])]
        ra = self.global_args.runtime_args
        ra.consumed_samples = int(ra.consumed_samples or 0) + self.sample_per_episode
        return merged
