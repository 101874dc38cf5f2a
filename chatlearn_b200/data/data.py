"""Dataset reading, the rollout data loader and the episode → train-batch stream.

Parity: chatlearn/data/data.py:33-386 (``read_data_path_list``,
``StreamDataset``, ``EpisodeReplayBuffer``, ``ReplaySampleManager``,
``RLHFDataLoader``).  The reference's ``StreamDataset`` is a Ray actor fed by
Ray queues of object refs; here every rank holds the episode's sample list in
process (roles share one process per GPU), so the stream is a plain object and
the "queue" is a list of rollout batches.
"""
import json
import math
import random
from abc import ABC, abstractmethod
from typing import Any, Callable, Dict, List, Optional, Sequence

from chatlearn_b200.utils.utils import even_slice


def read_data_path_list(data_path_list, mode: str = "jsonl") -> List[List[Dict[str, Any]]]:
    """Read one dataset per path.  Paths may be a list or a comma-separated
    string; ``.jsonl``, ``.json`` and ``.parquet`` files are recognised by suffix."""
    if isinstance(data_path_list, str):
        data_path_list = [p for p in data_path_list.split(",") if p]
    out = []
    for path in data_path_list:
        suffix = path.rsplit(".", 1)[-1].lower() if "." in path else mode
        if suffix == "jsonl":
            with open(path, "r", encoding="utf-8") as f:
                out.append([json.loads(line) for line in f if line.strip()])
        elif suffix == "json":
            with open(path, "r", encoding="utf-8") as f:
                text = f.read()
            try:
                rows = json.loads(text)
            except json.JSONDecodeError:
                # dataset exporters write one JSON object per line into ".json" files
                rows = [json.loads(line) for line in text.splitlines() if line.strip()]
            out.append(rows if isinstance(rows, list) else [rows])
        elif suffix == "parquet":
            import pandas as pd
            out.append(pd.read_parquet(path).to_dict(orient="records"))
        else:
            raise ValueError(f"unsupported dataset file '{path}'")
    return out


class RLHFDataLoader:
    """Iterates episodes of prompt samples for one rollout replica.

    ``datasets``: list of indexable datasets; ``sampler`` yields per-episode
    lists of ``(dataset id, row, position)``.  Every sample is stamped with
    ``prompt_uid`` (shared by the copies of one prompt inside an episode) and a
    globally unique ``uid`` (data.py:372-386)."""

    def __init__(self, datasets: Sequence, sampler, collate_fn: Optional[Callable] = None,
                 add_uid: bool = True, data_parallel_rank: int = 0, data_parallel_size: int = 1,
                 num_inference_per_prompt: int = 1, vllm_prompt_key: str = "prompt"):
        self.datasets = datasets
        self.sampler = sampler
        self.collate_fn = collate_fn
        self.add_uid = add_uid
        self.dp_rank, self.dp_size = data_parallel_rank, data_parallel_size
        self.n = num_inference_per_prompt
        self.key = vllm_prompt_key
        self._uid = 0

    def __iter__(self):
        while True:
            for batch_idx in iter(self.sampler):
                batch = []
                for ds, row, _pos in batch_idx:
                    sample = dict(self.datasets[ds][row])
                    if self.add_uid:
                        sample["prompt_uid"] = f"{ds}_{row}"
                        sample["uid"] = self._uid * self.dp_size + self.dp_rank
                        self._uid += 1
                    batch.append(sample)
                yield self.collate_fn(batch) if self.collate_fn else batch


class EpisodeReplayBuffer:
    """The samples of one episode."""

    def __init__(self, episode_id: int, queue: Optional[List[List[Dict]]] = None,
                 buffer: Optional[List[Dict]] = None):
        self._episode_id = episode_id
        self._queue = list(queue) if queue is not None else []
        self._buffer: List[Dict] = list(buffer) if buffer is not None else []

    def queue_not_empty(self) -> bool:
        return bool(self._queue)

    def add_raw_batch(self):
        if self._queue:
            self._buffer.extend(self._queue.pop(0))

    def sync(self):
        while self._queue:
            self.add_raw_batch()

    def shuffle(self, seed=None):
        rnd = random.Random(seed if seed is not None else self._episode_id)
        rnd.shuffle(self._buffer)

    def get_samples(self, start: int, end: int) -> List[Dict]:
        return self._buffer[start:end]

    def total_train_tokens(self) -> int:
        tot = 0
        for s in self._buffer:
            tot += int(s.get("prompt_token_length", 0)) + int(s.get("response_token_length", 0))
        return tot

    @property
    def buffer(self):
        return self._buffer

    @property
    def episode_id(self):
        return self._episode_id

    def __len__(self):
        return len(self._buffer)


class ReplaySampleManager(ABC):
    """User hook: turn the window of recent episode buffers into the list of
    samples to train on (GRPO plugs its advantage computation in here)."""

    def __init__(self, args=None):
        self.args = args
        self._metric_prefix = "replay"
        self._metric_list = []

    @abstractmethod
    def __call__(self, episode_replay_buffers: List[EpisodeReplayBuffer]) -> List[Dict]:
        ...

    def get_and_clear_metrics(self):
        from chatlearn_b200.utils.utils import map_reduce_metrics
        if not self._metric_list:
            return self._metric_prefix, {}
        m = map_reduce_metrics(self._metric_list)
        self._metric_list = []
        return self._metric_prefix, m


class StreamDataset:
    """Turns the rollout output of an episode into train mini-batches.

    Slicing rule (data.py:154-176): the episode buffer is cut into ``dp_size``
    even slices first, then each slice into ``num_minibsz`` even mini-batches;
    ``next()`` returns them in (dp rank, iteration) order, so mini-batch
    ``r * num_minibsz + i`` is what DP rank ``r`` trains on at step ``i``."""

    def __init__(self, data_loader_type: str, num_minibsz: int,
                 replay_sample_manager: Optional[ReplaySampleManager], micro_batch_size: int,
                 max_replay_episode: int = 0, replay_episode_offset: int = 0):
        self._dynamic = data_loader_type != "fixed"
        self.num_minibsz = num_minibsz
        self.batch_size = micro_batch_size
        self.dp_size: Optional[int] = None
        self._max_replay_episode = math.inf if max_replay_episode < 0 else max_replay_episode
        self._replay_episode_offset = replay_episode_offset
        self._episode_replay_buffers: List[EpisodeReplayBuffer] = []
        self.replay_sample_manager = replay_sample_manager
        self.replay_buffer: Optional[EpisodeReplayBuffer] = None
        self._total_samples = 0
        self._iter = None
        self._has_next = False

    def set_dp_size(self, dp_size: int):
        self.dp_size = dp_size

    def set_dataset(self, queue: List[List[Dict]], episode_id: int, sample_per_episode: int = -1):
        buf = EpisodeReplayBuffer(episode_id, queue=queue)
        buf.sync()
        if self._max_replay_episode > 0 and episode_id >= self._replay_episode_offset:
            self._episode_replay_buffers.append(buf)
            if len(self._episode_replay_buffers) > self._max_replay_episode:
                self._episode_replay_buffers.pop(0)
            if self.replay_sample_manager is not None:
                samples = self.replay_sample_manager(self._episode_replay_buffers)
            else:
                samples = buf.buffer
            self.replay_buffer = EpisodeReplayBuffer(episode_id, buffer=samples)
        else:
            self.replay_buffer = buf
        self._total_samples = len(self.replay_buffer)
        if sample_per_episode != -1 and self.replay_sample_manager is None:
            assert self._total_samples == sample_per_episode, \
                f"episode produced {self._total_samples} samples, expected {sample_per_episode}"
        self._iter = iter(self)
        self._has_next = True

    def boundaries(self) -> List[int]:
        assert self.dp_size is not None, "set_dp_size() must be called before fetching"
        dp = even_slice(self._total_samples, self.dp_size)
        cuts = [s + m for s, e in zip(dp[:-1], dp[1:])
                for m in even_slice(e - s, self.num_minibsz)[:-1]]
        cuts.append(self._total_samples)
        return cuts

    def __iter__(self):
        cuts = self.boundaries()
        for s, e in zip(cuts[:-1], cuts[1:]):
            yield self.replay_buffer.get_samples(s, e)
        self._has_next = False

    def minibatch(self, dp_rank: int, iteration: int) -> List[Dict]:
        """Random access to the mini-batch of (dp rank, iteration)."""
        cuts = self.boundaries()
        k = dp_rank * self.num_minibsz + iteration
        return self.replay_buffer.get_samples(cuts[k], cuts[k + 1])

    def shuffle(self):
        self.replay_buffer.shuffle()
        self._iter = iter(self)
        self._has_next = True

    def next(self):
        return next(self._iter)

    def has_next(self):
        return self._has_next

    def get_total_train_tokens(self):
        return self.replay_buffer.total_train_tokens()

    def episode_replay_buffers(self):
        return self._episode_replay_buffers

    def num_iteration(self):
        return self.num_minibsz

    def total_samples(self):
        return self._total_samples

    def batch_per_episode(self):
        return math.ceil(self._total_samples / self.batch_size)

    def get_and_clear_metrics(self):
        if self.replay_sample_manager is None:
            return "no replay", {}
        return self.replay_sample_manager.get_and_clear_metrics()
