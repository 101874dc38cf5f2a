"""Deterministic, resumable prompt samplers.

Parity: chatlearn/data/sampler.py:149-363 (``RLHFSingleSampler``,
``MultiDatasetSampler``) and :22-147 (legacy ``SingleDataSampler`` /
``EpisodeDataSampler``).  Behaviour kept:

* every episode draws ``sample_per_episode / n`` prompts, where datasets are
  mixed by ``data_ratio`` in a repeating pattern ``[0]*r0 + [1]*r1 + …``;
* each dataset is walked through an epoch-seeded permutation
  (``seed + epoch``), so a sampler rebuilt with the same ``consumed_samples``
  continues with the same sequence;
* each prompt is repeated ``n`` times, interleaved (``p0 p0 … p1 p1``) or
  block-repeated when ``data_rerank`` (``p0 p1 … p0 p1 …``) so that copies of a
  prompt land on different replicas;
* the episode's index list is cut into even slices per data-parallel rank.

The state here is a single integer per dataset (prompts consumed), which makes
the resume rule explicit instead of being spread over offset/epoch fields.
"""
from typing import Iterator, List, Optional, Sequence, Tuple

import torch

from chatlearn_b200.utils.utils import even_slice

Index = Tuple[int, int, int]  # (dataset id, row in dataset, prompt position in the episode)


class EpochPermutation:
    """Walks one dataset through per-epoch permutations.

    ``mode``: ``cycle`` wraps into the next epoch inside one request,
    ``retain`` returns the (short) tail of the epoch, ``drop`` skips a tail that
    cannot fill the request."""

    def __init__(self, size: int, consumed: int = 0, shuffle: bool = True, seed: int = 0,
                 mode: str = "cycle", batch: int = 1):
        assert size > 0, "empty dataset"
        assert mode in ("cycle", "retain", "drop")
        self.size, self.shuffle, self.seed, self.mode = size, shuffle, seed, mode
        usable = (size // batch) * batch if mode == "drop" else size
        assert usable > 0, "drop mode needs a dataset at least as large as one batch"
        self.epoch, self.cursor = divmod(consumed, usable)
        self._perm_epoch = None
        self._perm: List[int] = []

    def _order(self) -> List[int]:
        if self._perm_epoch != self.epoch:
            if self.shuffle:
                g = torch.Generator()
                g.manual_seed(self.epoch + self.seed)
                self._perm = torch.randperm(self.size, generator=g).tolist()
            else:
                self._perm = list(range(self.size))
            self._perm_epoch = self.epoch
        return self._perm

    def _advance_epoch(self):
        self.epoch += 1
        self.cursor = 0

    def take(self, num: int) -> List[int]:
        out: List[int] = []
        if self.mode == "drop":
            assert num <= self.size
            if num > self.size - self.cursor:
                self._advance_epoch()
            out = self._order()[self.cursor:self.cursor + num]
            self.cursor += num
            return out
        if self.mode == "retain":
            if num > self.size - self.cursor:
                out = self._order()[self.cursor:]
                self._advance_epoch()
            else:
                out = self._order()[self.cursor:self.cursor + num]
                self.cursor += num
            return out
        while num >= self.size - self.cursor:
            out.extend(self._order()[self.cursor:])
            num -= self.size - self.cursor
            self._advance_epoch()
        out.extend(self._order()[self.cursor:self.cursor + num])
        self.cursor += num
        return out


# name kept for users of the reference API
RLHFSingleSampler = EpochPermutation


class MultiDatasetSampler:
    """Yields, per episode, this DP rank's list of ``(dataset, row, position)``."""

    def __init__(self, dataset_sizes: Sequence[int], sample_per_episode: int,
                 data_ratio=None, consumed_samples: int = 0, num_inference_per_prompt: int = 1,
                 shuffle: bool = True, seed: Optional[int] = None, is_eval: bool = False,
                 init_shuffle_prompt: int = 0, data_parallel_rank: int = 0,
                 data_parallel_size: int = 1, drop_last: str = "cycle", data_rerank: bool = False):
        self.dataset_sizes = list(dataset_sizes)
        self.sample_per_episode = sample_per_episode
        self.n = num_inference_per_prompt
        self.is_eval = is_eval
        self.dp_rank, self.dp_size = data_parallel_rank, data_parallel_size
        self.data_rerank = data_rerank
        nds = len(self.dataset_sizes)
        self.mode = drop_last if nds == 1 else "cycle"
        assert init_shuffle_prompt == 0, "init_shuffle_prompt 1/2 are not supported"
        assert consumed_samples % self.n == 0, \
            "consumed_samples must be a multiple of num_inference_per_prompt"
        assert sample_per_episode % self.n == 0, \
            "sample_per_episode must be a multiple of num_inference_per_prompt"
        if is_eval:
            return
        if not data_ratio:
            ratio = [1] * nds
        elif isinstance(data_ratio, int):
            ratio = [data_ratio] * nds
        else:
            ratio = list(data_ratio)
            assert len(ratio) == nds, f"data_ratio has {len(ratio)} entries for {nds} datasets"
        self.data_ratio = ratio
        # mixing pattern: dataset id of the k-th prompt is pattern[k % len(pattern)]
        self.pattern = [d for d, r in enumerate(ratio) for _ in range(r)]
        prompts_done = consumed_samples // self.n
        self.pattern_pos = prompts_done % len(self.pattern)
        full, rem = divmod(prompts_done, len(self.pattern))
        consumed_each = [r * full for r in ratio]
        for d in self.pattern[:rem]:
            consumed_each[d] += 1
        seed = 0 if seed is None else seed
        per_episode = sample_per_episode // self.n
        self.walkers = [
            EpochPermutation(self.dataset_sizes[d], consumed_each[d], shuffle, seed, self.mode,
                             batch=per_episode if nds == 1 else ratio[d])
            for d in range(nds)]

    def _repeat(self, items: List[Index]) -> List[Index]:
        if self.data_rerank:
            return items * self.n
        return [it for it in items for _ in range(self.n)]

    def _eval_indices(self) -> List[Index]:
        flat: List[Index] = []
        for d, size in enumerate(self.dataset_sizes):
            base = len(flat)
            flat.extend((d, j, base + j) for j in range(size))
        b = even_slice(len(flat), self.dp_size)
        return flat[b[self.dp_rank]:b[self.dp_rank + 1]]

    def _draw_prompts(self, num: int) -> List[Index]:
        if len(self.walkers) == 1:
            rows = self.walkers[0].take(num)
            return [(0, r, i) for i, r in enumerate(rows)]
        out: List[Index] = []
        while len(out) < num:
            d = self.pattern[self.pattern_pos]
            # take the run of consecutive identical dataset ids in one request
            run = 1
            while (self.pattern_pos + run < len(self.pattern) and len(out) + run < num
                   and self.pattern[self.pattern_pos + run] == d):
                run += 1
            rows = self.walkers[d].take(run)
            base = len(out)
            out.extend([(d, r, base + i) for i, r in enumerate(rows)])
            self.pattern_pos = (self.pattern_pos + run) % len(self.pattern)
        return out

    def __iter__(self) -> Iterator[List[Index]]:
        if self.is_eval:
            yield self._eval_indices()
            return
        per_episode = self.sample_per_episode // self.n
        while True:
            episode = self._repeat(self._draw_prompts(per_episode))
            b = even_slice(len(episode), self.dp_size)
            yield episode[b[self.dp_rank]:b[self.dp_rank + 1]]


class SingleDataSampler:
    """Plain sequential DP sampler (legacy API, chatlearn/data/sampler.py:22-75)."""

    def __init__(self, total_samples, consumed_samples, micro_batch_size, data_parallel_rank,
                 data_parallel_size, dynamic_batch_size_flag=False, drop_last=False):
        assert total_samples > 0 and micro_batch_size > 0
        assert 0 <= data_parallel_rank < data_parallel_size
        self.total, self.consumed = total_samples, consumed_samples
        self.mbs, self.rank, self.size = micro_batch_size, data_parallel_rank, data_parallel_size
        self.drop_last = drop_last
        self.dynamic = dynamic_batch_size_flag

    def __len__(self):
        return self.total

    def __iter__(self):
        step = self.mbs * self.size
        batch = []
        for idx in range(self.consumed, self.total):
            batch.append(idx)
            if len(batch) == step:
                yield batch[self.rank * self.mbs:(self.rank + 1) * self.mbs]
                batch = []
        if batch and not self.drop_last:
            if self.dynamic:
                b = even_slice(len(batch), self.size)
                yield batch[b[self.rank]:b[self.rank + 1]]
            else:
                yield batch[self.rank * self.mbs:(self.rank + 1) * self.mbs]


class EpisodeDataSampler:
    """Episode-aware cyclic sampler (legacy API, chatlearn/data/sampler.py:77-147).

    Walks ``range(total_samples)`` in batches of ``micro_batch_size * dp_size``;
    a batch that would cross the end of the dataset wraps to the beginning
    (unless ``drop_last``), and an episode boundary (``sample_per_episode``)
    flushes a short batch so no batch straddles two episodes."""

    def __init__(self, total_samples, consumed_samples, micro_batch_size, data_parallel_rank,
                 data_parallel_size, sample_per_episode, drop_last=False):
        assert total_samples > 0 and micro_batch_size > 0
        self.total, self.consumed = total_samples, consumed_samples
        self.mbs, self.rank, self.size = micro_batch_size, data_parallel_rank, data_parallel_size
        self.sample_per_episode = sample_per_episode
        self.drop_last = drop_last
        self.episode_offset = consumed_samples % sample_per_episode if sample_per_episode else 0

    def _mine(self, batch):
        b = even_slice(len(batch), self.size) if len(batch) != self.mbs * self.size else None
        if b is None:
            return batch[self.rank * self.mbs:(self.rank + 1) * self.mbs]
        return batch[b[self.rank]:b[self.rank + 1]]

    def __iter__(self):
        step = self.mbs * self.size
        batch = []
        pos = self.consumed % self.total
        in_episode = self.episode_offset
        while True:
            batch.append(pos)
            pos += 1
            in_episode += 1
            if pos == self.total:
                pos = 0
                if self.drop_last and len(batch) < step:
                    batch = []
                    in_episode = in_episode - in_episode % step
            flush = len(batch) == step
            if self.sample_per_episode and in_episode >= self.sample_per_episode:
                flush = bool(batch)
                in_episode = 0
            if flush:
                yield self._mine(batch)
                batch = []
