"""Group-normalised advantages.

Parity: chatlearn/algorithm/grpo_utils/advantage_compute.py:18-44.  Rewards are
accumulated per ``prompt_uid`` across episodes; every sample of the current
episode gets ``A = (r - mean) / (std + 1e-5)`` (population standard deviation)
over the rewards seen so far for its prompt, and the whole episode buffer is
returned.  With partial rollout a prompt's samples can arrive over several
episodes: early arrivals are trained at once against the statistics of what has
arrived, later ones against the fuller group.  A prompt's rewards are dropped
once ``num_inference_per_prompt`` of them have been seen, so the table cannot
grow beyond the prompts that are still in flight.
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
        self.rule_reward_buffer: Dict[str, List[float]] = defaultdict(list)

    def __call__(self, episode_replay_buffers) -> List[Dict]:
        buf = episode_replay_buffers[-1].buffer
        for s in buf:
            self.rule_reward_buffer[s["prompt_uid"]].append(float(s["rule_reward"]))
        stats = {}
        for uid in {s["prompt_uid"] for s in buf}:
            r = np.asarray(self.rule_reward_buffer[uid], dtype=np.float64)
            stats[uid] = (r.mean(), r.std(), bool((r == 1).all()), bool((r == 0).all()))
        all_correct = all_wrong = 0
        for s in buf:
            mean, std, ones, zeros = stats[s["prompt_uid"]]
            s["advantages"] = float((float(s["rule_reward"]) - mean) / (std + 1e-5))
            all_correct += ones
            all_wrong += zeros
        for uid in [u for u, v in self.rule_reward_buffer.items() if len(v) >= self.n]:
            del self.rule_reward_buffer[uid]
        if buf:
            self._metric_list.append({"all_correct_ratio": all_correct / len(buf),
                                      "all_wrong_ratio": all_wrong / len(buf)})
        return buf
