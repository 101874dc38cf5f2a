"""Group-normalised advantages.

Parity: chatlearn/algorithm/grpo_utils/advantage_compute.py:18-44.  Samples are
grouped by ``prompt_uid``; ``A = (r - mean) / (std + 1e-5)`` with the population
standard deviation.  With partial rollout a prompt's samples can arrive over
several episodes, so groups are keyed across the replay window and only complete
groups (``num_inference_per_prompt`` samples) are released.
"""
from collections import defaultdict
from typing import Dict, List

import numpy as np

from chatlearn_b200.data.data import ReplaySampleManager


class AdvantageComputer(ReplaySampleManager):
    def __init__(self, num_inference_per_prompt: int):
        super().__init__()
        self.n = num_inference_per_prompt
        self._metric_prefix = "advantage_compute"
        self.pending: Dict[str, List[Dict]] = defaultdict(list)

    def __call__(self, episode_replay_buffers) -> List[Dict]:
        buf = episode_replay_buffers[-1].buffer
        for s in buf:
            self.pending[s["prompt_uid"]].append(s)
        out: List[Dict] = []
        all_correct = all_wrong = groups = 0
        for uid in list(self.pending):
            grp = self.pending[uid]
            if len(grp) < self.n:
                continue
            r = np.array([float(s["rule_reward"]) for s in grp], dtype=np.float64)
            mean, std = r.mean(), r.std()
            for s, ri in zip(grp, r):
                s["advantages"] = float((ri - mean) / (std + 1e-5))
            groups += 1
            all_correct += int((r > 0).all() and std == 0)
            all_wrong += int((r <= 0).all() and std == 0)
            out.extend(grp)
            del self.pending[uid]
        if groups:
            self._metric_list.append({"all_correct_ratio": all_correct / groups,
                                      "all_wrong_ratio": all_wrong / groups})
        return out
