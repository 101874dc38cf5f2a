"""Partial (multi-round, truncated) rollout.

Parity: chatlearn/algorithm/grpo_utils/partial_rollout_manager.py:11-133.  Long
generations are cut into rounds: round ``i`` may add at most
``max_response_tokens_length * rollout_ratio[i]`` tokens; a sample that used its
whole round budget is carried over (its tokens so far become the next round's
input), a sample that stopped early or reached the last round is finished.  A
prompt's finished samples are released for training once more than
``mini_response_per_prompt`` of them exist.  The manager is a CPU role with global
state, so it runs on one rank (``num_cpu: 1``) and sees the whole episode.
"""
import random
from collections import defaultdict
from typing import Any, Dict, List

import numpy as np

from chatlearn_b200.models.base_module import BaseModule


class PartialRolloutManager(BaseModule):
    whole_batch = True        # the executor hands over the episode in one call, not in generation batches

    def setup(self):
        self._metric_prefix = "partial_rollout_manager"
        ma = self.module_args
        pol = self.global_args.models.policy
        self.max_rollout_round = int(ma.max_rollout_round)
        self.max_token_per_round = [int(pol.max_response_tokens_length * r) for r in ma.rollout_ratio]
        self.num_inference_per_prompt = int(pol.num_inference_per_prompt)
        self.mini_response_per_prompt = int(ma.mini_response_per_prompt)
        assert self.mini_response_per_prompt < self.num_inference_per_prompt, \
            "mini_response_per_prompt must be less than num_inference_per_prompt"
        self.unfinished: Dict[Any, Dict] = {}                       # uid -> sample still generating
        self.finished_by_prompt: Dict[str, List[Dict]] = defaultdict(list)
        self.finished_count: Dict[str, int] = defaultdict(int)
        self._episode = 0
        self._rnd = random.Random(int(getattr(ma, "seed", 1234)))
        self._round_metrics: Dict[str, float] = {}

    def before_episode(self):
        self._episode += 1

    # ---- flow node 1: which samples go to the rollout engine this episode ----
    def get_sample_for_rollout(self, data: List[Dict[str, Any]], iteration: int = 0, **kwargs):
        for s in data:
            s["rollout_round"] = 0
            s["max_generate_token_length"] = self.max_token_per_round[0]
            s.setdefault("start_episode", self._episode)
            self.unfinished[s["uid"]] = s
        batch = list(self.unfinished.values())
        self._rnd.shuffle(batch)
        rounds = {f"round_{i}_samples": 0 for i in range(self.max_rollout_round)}
        for s in batch:
            rounds[f"round_{s['rollout_round']}_samples"] += 1
        self._round_metrics = dict(rounds)
        return batch

    def is_finished(self, s: Dict[str, Any]) -> bool:
        return s["response_token_length_round"] < s["max_generate_token_length"] \
            or s["rollout_round"] == self.max_rollout_round

    # ---- flow node 2: merge the round's generations, release complete prompts ----
    def post_process_rollout_results(self, results: List[Dict[str, Any]], iteration: int = 0, **kwargs):
        per_round = {i: [] for i in range(self.max_rollout_round)}
        for r in results:
            uid = r["uid"]
            kept = self.unfinished[uid]
            prev_resp = int(kept.get("response_token_length", 0)) if kept.get("rollout_round", 0) > 0 else 0
            total_resp = int(r["response_token_length"])            # the engine reports prompt-relative length
            this_round = total_resp - prev_resp
            rnd = int(r["rollout_round"])
            per_round[min(rnd - 1, self.max_rollout_round - 1)].append(this_round)
            kept.update({
                "str_outputs": r.get("str_outputs", ""), "rollout_round": rnd,
                "response_token_length": total_resp, "response_token_length_round": this_round,
                "prompt_token_length": r["prompt_token_length"], "all_tokens": r["all_tokens"],
                "input_ids": r["all_tokens"].tolist(),
                "max_generate_token_length": kept["max_generate_token_length"],
            })
            for k in ("rollout_logprobs", "finish_reason", "all_token_length"):
                if k in r:
                    kept[k] = r[k]
            if self.is_finished(kept):
                del self.unfinished[uid]
                self.finished_by_prompt[kept["prompt_uid"]].append(kept)
                self.finished_count[kept["prompt_uid"]] += 1
            else:
                kept["max_generate_token_length"] = self.max_token_per_round[rnd]
        train = []
        for key in list(self.finished_by_prompt):
            if self.finished_count[key] > self.mini_response_per_prompt:
                train.extend(self.finished_by_prompt.pop(key))
                if self.finished_count[key] == self.num_inference_per_prompt:
                    del self.finished_count[key]
        self._rnd.shuffle(train)
        m = dict(self._round_metrics)
        for i, lens in per_round.items():
            arr = np.array(lens or [0])
            m[f"round_{i}_response_mean"], m[f"round_{i}_response_max"], m[f"round_{i}_response_min"] = \
                float(arr.mean()), float(arr.max()), float(arr.min())
        m["total_valid_tokens"] = sum(int(d["response_token_length"]) + int(d["prompt_token_length"]) for d in train)
        m["num_train_samples"] = len(train)
        self._metric_list.append(m)
        return train
