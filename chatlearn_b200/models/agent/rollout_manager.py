"""Rollout manager: front of the agent/async rollout path.

Parity: chatlearn/models/agent/rollout_manager.py:30-177.  The reference manager is
a CPU actor that feeds requests one by one to async engines (``max_concurrent_per_engine``
in flight each), collects them as they finish, and finally re-orders the samples so
that every trainer data-parallel rank gets about the same number of tokens.

In this SPMD runtime the manager is co-located with the rollout role: it takes the
placement and data-parallel geometry of the engine module it fronts, its
``forward_step`` runs on every engine replica over that replica's share of the
episode (the engine's continuous batching, capped at ``max_concurrent_per_engine``
running sequences, plays the part of the in-flight window), and the token balancing
runs in ``post_gather`` on the complete sample list, identically on all ranks.
"""
import heapq
from typing import Dict, List

from chatlearn_b200.models.base_module import BaseModule


def balance_by_tokens(data: List[Dict], dp_size: int, batch_size: float, key: str = "all_token_length") -> List[Dict]:
    """Greedy longest-first packing into ``dp_size`` groups of ``batch_size`` samples;
    the result is the groups laid end to end (rollout_manager.py:68-99)."""
    order = sorted(range(len(data)), key=lambda i: (-int(data[i][key]), i))
    heap = [(0, g) for g in range(dp_size)]
    heapq.heapify(heap)
    groups: List[List[int]] = [[] for _ in range(dp_size)]
    closed: List[int] = []
    for i in order:
        if not heap:
            break
        total, g = heapq.heappop(heap)
        groups[g].append(i)
        if len(groups[g]) >= batch_size:
            closed.append(g)
        else:
            heapq.heappush(heap, (total + int(data[i][key]), g))
    while heap:
        closed.append(heapq.heappop(heap)[1])
    return [data[i] for g in closed for i in groups[g]]


class RolloutManager(BaseModule):
    whole_batch = True        # a replica's whole share at once; the engine batches continuously

    def __init__(self, name: str = "rollout_manager", engine_module=None, args=None, replica_id: int = 0):
        super().__init__(name, args, replica_id)
        ma = self.module_args
        assert int(ma.num_cpu) // max(int(getattr(ma, "cpu_per_process", 1) or 1), 1) == 1, \
            "there is exactly one rollout manager"
        self.engine_module = engine_module
        self._metric_prefix = "rollout_manager"

    def attach(self, engine_module):
        self.engine_module = engine_module

    # ---- geometry: the manager lives where its engines live ----
    @property
    def is_member(self):
        return self.engine_module.is_member

    @property
    def data_parallel_size(self):
        return self.engine_module.data_parallel_size

    @property
    def data_parallel_rank(self):
        return self.engine_module.data_parallel_rank

    @property
    def is_data_leader(self):
        return self.engine_module.is_data_leader

    @property
    def is_replica_leader(self):
        return self.engine_module.is_replica_leader

    @property
    def replica_index(self):
        return self.engine_module.replica_index

    @property
    def num_replica(self):
        return self.engine_module.num_replica

    @property
    def loader_parallel_size(self):
        return self.engine_module.loader_parallel_size

    @property
    def is_colocate(self):
        return self.engine_module.is_colocate

    @property
    def residency_args(self):
        """The executor onloads/offloads around this role's nodes as it would around the engine's."""
        return self.engine_module.module_args.free_gpu_memory

    def setup(self):
        assert self.engine_module is not None, "RolloutManager needs the rollout module it fronts"
        assert not self.runtime_args.data_rerank, "data_rerank must be off when the rollout manager is used"
        ma = self.module_args
        eng = getattr(self.engine_module, "engine", None)
        if eng is not None and bool(ma.use_dynamic_load_blance):
            eng.max_num_seqs = min(eng.max_num_seqs, int(ma.max_concurrent_per_engine))

    def _forward(self, data: List[Dict], iteration: int, is_eval: bool):
        return self.engine_module.forward_step(data, iteration, is_eval=is_eval)

    def forward_step(self, data: List[Dict], iteration: int = 0, **kwargs):
        rets = self._forward(data, iteration, False)
        self._metric_list.extend(self.engine_module._metric_list)
        self.engine_module._metric_list = []
        return rets

    def eval_forward(self, data: List[Dict], iteration: int = 0, **kwargs):
        return self._forward(data, iteration, True)

    def post_gather(self, samples: List[Dict], func_name: str) -> List[Dict]:
        """Runs on every rank on the gathered episode: token-balance over trainer DP."""
        if func_name != "forward_step" or not samples:
            return samples
        tr = self.global_args.models.policy_trainer
        dp = max(int(getattr(tr, "replica_dp_size", 1) or 1) * int(getattr(tr, "num_replica", 1) or 1), 1)
        return balance_by_tokens(samples, dp, len(samples) / dp)

    def onload(self, **kw):
        self.engine_module.onload(**kw)

    def offload(self, **kw):
        self.engine_module.offload(**kw)
