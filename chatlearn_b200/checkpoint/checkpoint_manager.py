"""Data checkpoint: where the run is in the prompt stream.

Parity: chatlearn/checkpoint/checkpoint_manager.py:27-151 — same on-disk layout:
``{path}/replica{r}_step{iteration}/meta.pkl`` holding ``{episode, train_iteration,
consumed_samples, sample_per_episode, data_ratio}``, a
``latest_checkpointed_iteration.txt`` pointer, and pruning to the newest
``max_ckpt_nums`` checkpoints.
"""
import os
import pickle
import shutil
from typing import Dict, Optional

from chatlearn_b200.utils.logger import logger

LATEST = "latest_checkpointed_iteration.txt"


def path_to_replica_step(path: str):
    """'…/replica0_step12' → (0, 12)."""
    base = os.path.basename(path.rstrip("/"))
    rep, step = base.split("_")
    return int(rep.replace("replica", "")), int(step.replace("step", ""))


class CheckpointManager:
    def __init__(self, model, path: str, max_ckpt_nums: Optional[int] = None,
                 load_iteration: Optional[int] = None, config_to_check: Optional[Dict] = None):
        self._model = model
        self._path = path
        self._max = max_ckpt_nums
        self._load_iteration = load_iteration
        self._config_to_check = config_to_check or {}
        self._meta = None
        self._resumed = False

    def _dir(self, replica_id: int, iteration: int) -> str:
        return os.path.join(self._path, f"replica{replica_id}_step{iteration}")

    def _latest_file(self) -> str:
        return os.path.join(self._path, LATEST)

    def _get_checkpoint_path_name(self, replica_id, step):
        return self._dir(replica_id, step)

    def save_checkpoint(self, replica_id: int, train_iter: int, episode: int, consumed_samples: int):
        d = self._dir(replica_id, train_iter)
        os.makedirs(d, exist_ok=True)
        ra = self._model.runtime_args
        meta = {"episode": episode, "train_iteration": train_iter, "consumed_samples": consumed_samples,
                "sample_per_episode": ra.sample_per_episode, "data_ratio": ra.data_ratio}
        tmp = os.path.join(d, "meta.pkl.tmp")
        with open(tmp, "wb") as f:
            pickle.dump(meta, f)
        os.replace(tmp, os.path.join(d, "meta.pkl"))
        # every replica writes the same pointer; a per-writer temp name keeps the
        # rename atomic without the replicas racing on one temp file
        tmp_latest = f"{self._latest_file()}.tmp.{replica_id}.{os.getpid()}"
        with open(tmp_latest, "w", encoding="utf-8") as f:
            f.write(str(train_iter))
        os.replace(tmp_latest, self._latest_file())
        self._prune(replica_id)
        logger.info(f"saved data checkpoint {d}")

    def _prune(self, replica_id: int):
        if not self._max or self._max <= 0:
            return
        mine = []
        for name in os.listdir(self._path):
            if name.startswith(f"replica{replica_id}_step"):
                mine.append((path_to_replica_step(name)[1], name))
        mine.sort()
        for _, name in mine[:-self._max]:
            shutil.rmtree(os.path.join(self._path, name), ignore_errors=True)

    def resume_meta(self):
        return self._meta

    def resume(self) -> Optional[Dict]:
        if self._resumed:
            return self._meta
        self._resumed = True
        it = self._load_iteration
        if it is None:
            if not os.path.exists(self._latest_file()):
                return None
            with open(self._latest_file(), "r", encoding="utf-8") as f:
                it = int(f.read().strip())
        rep = getattr(self._model, "replica_index", 0)
        d = self._dir(rep, it)
        if not os.path.exists(os.path.join(d, "meta.pkl")):
            d = self._dir(0, it)       # replicas share the position in the stream
            if not os.path.exists(os.path.join(d, "meta.pkl")):
                return None
        with open(os.path.join(d, "meta.pkl"), "rb") as f:
            self._meta = pickle.load(f)
        for k, v in self._config_to_check.items():
            assert self._meta.get(k) == v, f"checkpoint {k}={self._meta.get(k)} differs from config {v}"
        logger.info(f"resuming data stream from {d}: {self._meta}")
        return self._meta
