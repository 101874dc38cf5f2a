"""Placement of model roles on ranks, colocation, and the parameter-sync choreography.

Parity: chatlearn/schedule/model_manager.py:81-406.  The reference creates
fractional-GPU Ray actors inside placement groups; with one process per GPU a
*placement* is simply the list of global ranks hosting a role:

* roles named in one ``runtime_args.colocation`` group share the same ranks and
  are time-sliced by the executor (onload/offload between phases);
* other GPU roles get disjoint rank ranges while the job has ranks left, and are
  packed into already-used ranges (largest first) when it does not — the packing
  rule of ``find_model_packing_strategy`` (model_manager.py:220-263);
* CPU roles (``num_cpu`` > 0) run data-parallel on every rank.
"""
from typing import Dict, List, Tuple


from chatlearn_b200.schedule.resource_manager import ResourceManager
from chatlearn_b200.utils.constant import TAG_KV_CACHE, TAG_WEIGHTS
from chatlearn_b200.utils.logger import logger


from chatlearn_b200.utils.trace import span  # noqa: E402


class ModelManager:
    def __init__(self, models, resource_manager: ResourceManager, global_args):
        self.local_models = list(models)
        self.resource_manager = resource_manager
        self.global_args = global_args
        self.runtime_args = global_args.runtime_args
        self._sync_pairs: List[Tuple] = []
        self.parameter_sync_groups: Dict[str, object] = {}
        self.placements: Dict[str, List[int]] = {}
        self.dist_models = self.local_models

    def set_parameter_sync(self, src_model, dst_model):
        self._sync_pairs.append((src_model, dst_model))

    # ------------------------------------------------------------------ placement
    @staticmethod
    def find_model_packing_strategy(models, total_gpu: int) -> List[List]:
        """Pack models into as few "rounds" of ``total_gpu`` GPUs as possible
        (first-fit decreasing).  A:8, B:4, C:4 on 8 GPUs → [[A], [B, C]]."""
        order = sorted(models, key=lambda m: m.total_gpu, reverse=True)
        rounds: List[List] = []
        free: List[int] = []
        for m in order:
            assert m.total_gpu <= total_gpu, \
                f"{m.name} needs {m.total_gpu} GPUs, the job has {total_gpu}"
            for i, f in enumerate(free):
                if m.total_gpu <= f:
                    rounds[i].append(m)
                    free[i] -= m.total_gpu
                    break
            else:
                rounds.append([m])
                free.append(total_gpu - m.total_gpu)
        return rounds

    def compute_placements(self) -> Dict[str, List[int]]:
        W = self.resource_manager.total_slots
        by_name = {m.name: m for m in self.local_models}
        groups: List[List] = []
        seen = set()
        coloc = self.runtime_args.colocation or []
        if coloc and isinstance(coloc[0], str):
            coloc = [coloc]
        for names in coloc:
            grp = [by_name[n] for n in names if n in by_name and by_name[n].total_gpu > 0]
            if grp:
                gpus = {m.total_gpu for m in grp}
                assert len(gpus) == 1, f"colocated models must use the same number of GPUs: {names}"
                for m in grp:
                    m.set_colocate(len(grp) > 1)
                    seen.add(m.name)
                groups.append(grp)
        for m in self.local_models:
            if m.total_gpu > 0 and m.name not in seen:
                groups.append([m])
        # a group behaves like one model needing group[0].total_gpu ranks
        class _G:  # noqa: D401  (tiny adaptor for the packing routine)
            def __init__(self, grp):
                self.grp, self.total_gpu, self.name = grp, grp[0].total_gpu, grp[0].name
        rounds = self.find_model_packing_strategy([_G(g) for g in groups], W)
        if len(rounds) > 1:
            logger.info(f"GPU demand exceeds {W} ranks: roles are time-sliced over {len(rounds)} rounds")
        placements: Dict[str, List[int]] = {}
        for rnd in rounds:
            cursor = 0
            for g in rnd:
                ranks = list(range(cursor, cursor + g.total_gpu))
                cursor += g.total_gpu
                for m in g.grp:
                    placements[m.name] = ranks
                    if len(rounds) > 1:
                        m.set_colocate(True)
        for m in self.local_models:
            if m.total_gpu == 0:
                # CPU roles run data-parallel on the first ``num_cpu`` ranks (a role with
                # global state, e.g. a rollout manager, asks for one)
                placements[m.name] = list(range(max(1, min(W, int(m.total_cpu or W)))))
        return placements

    def create_dist_models(self):
        self.placements = self.compute_placements()
        me = self.resource_manager.rank
        for m in self.local_models:
            m.placement = self.placements[m.name]
            m.role_rank = m.placement.index(me) if me in m.placement else -1
            # the role's bundles (ranks per node, with the node's share of CPU cores): what the reference keeps as
            # a Ray placement group per model
            self.resource_manager.reserve(m.name, m.placement)
        return self.local_models

    # ------------------------------------------------------------------ parameter sync
    def build_parameter_group(self):
        from chatlearn_b200.synchronizer.parameter_sync import ParameterSyncGroup
        for src, dst in self._sync_pairs:
            key = f"{src.name}->{dst.name}"
            mode = str(getattr(dst.module_args, "sync_mode", "auto"))
            self.parameter_sync_groups[key] = ParameterSyncGroup(
                src, dst, mode=mode, bucket_size_mb=float(getattr(self.runtime_args, "bucket_size_mb_in_memory_manager", 1024)))

    def sync_parameters(self, episode_offset: int = 0, requires_grad=None, validate: bool = False):
        """onload trainer weights → onload rollout weights → sync → offload trainer →
        onload rollout KV cache (model_manager.py:169-195)."""
        ms = {}
        for key, grp in self.parameter_sync_groups.items():
            src, dst = grp.src, grp.dst
            freq = int(getattr(dst.module_args, "sync_frequency", 1) or 1)
            if episode_offset % freq != 0:
                continue
            with span("sync.src_onload"):
                if src.is_member:
                    src.onload(to_onload_weights=True, to_build_grad_buffers=False,
                               to_onload_optimizer_states=False)
            with span("sync.dst_onload_weights"):
                if dst.is_member:
                    dst.onload(tags=[TAG_WEIGHTS])
            with span("sync.copy"):
                ms[key] = grp.sync()
            with span("sync.src_offload"):
                if src.is_member and src.is_colocate:
                    src.offload()
            with span("sync.dst_onload_kv"):
                if dst.is_member:
                    dst.onload(tags=[TAG_KV_CACHE])
        return ms

    def clean(self):
        for m in self.local_models:
            m.terminate()
