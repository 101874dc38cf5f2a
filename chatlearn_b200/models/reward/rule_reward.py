"""Rule-based reward role (CPU).

Parity: chatlearn/models/reward/rule_reward.py:59-85: every sample gets
``rule_reward`` from the scorer selected by its ``data_source`` and keeps
``eval_source`` for the evaluator.  Besides the reference's MATH and geo3k
scorers the synthetic benchmark rewards (``mod7``, ``hash30``) are registered;
they score response token ids instead of text.
"""
from typing import Callable, Dict, List

import torch

from chatlearn_b200.data.synthetic import SYNTHETIC_REWARDS
from chatlearn_b200.models.base_module import BaseModule
from chatlearn_b200.utils.rule_reward_score import geo3k, math


class RuleReward(BaseModule):
    def __init__(self, name: str = "reward", args=None, replica_id: int = 0):
        super().__init__(name, args, replica_id)
        self._metric_prefix = "rule_reward"
        self.text_scorers: Dict[str, Callable[[str, str], float]] = {
            "openai/gsm8k": math.compute_score, "DigitalLearningGmbH/MATH-lighteval": math.compute_score,
            "aime24": math.compute_score, "aime25": math.compute_score, "math": math.compute_score,
            "hiyouga/geometry3k": geo3k.compute_score, "geo3k": geo3k.compute_score,
        }
        self.token_scorers = dict(SYNTHETIC_REWARDS)
        self.default_synthetic = str(getattr(self.module_args, "synthetic_reward", "hash30"))

    def register_scorer(self, data_source: str, fn: Callable, on_tokens: bool = False):
        (self.token_scorers if on_tokens else self.text_scorers)[data_source] = fn

    def select_rule_reward_score_fn(self, data_source: str):
        if data_source in self.text_scorers:
            return self.text_scorers[data_source], False
        if data_source in self.token_scorers:
            return self.token_scorers[data_source], True
        if data_source.startswith("synthetic"):
            key = data_source.split(":", 1)[1] if ":" in data_source else self.default_synthetic
            return self.token_scorers[key], True
        raise NotImplementedError(f"no rule reward for data_source '{data_source}'")

    def _score(self, sample: Dict) -> float:
        fn, on_tokens = self.select_rule_reward_score_fn(sample.get("data_source", ""))
        if on_tokens:
            toks = sample["all_tokens"]
            pl = int(sample["prompt_token_length"])
            resp = toks[pl:pl + int(sample["response_token_length"])]
            return float(fn(resp.tolist() if isinstance(resp, torch.Tensor) else list(resp)))
        return float(fn(sample.get("str_outputs", ""), sample.get("ground_truth", "")))

    def forward_step(self, data_list: List[Dict], iteration: int = 0, is_eval: bool = False, **kw):
        scores = []
        for s in data_list:
            r = self._score(s)
            s["rule_reward"] = r
            s["eval_source"] = s.get("data_source", "")
            scores.append(r)
        if scores and not is_eval:
            self._metric_list.append({"train_reward_score": sum(scores) / len(scores)})
        return data_list

    def eval_forward(self, data_list, iteration: int = 0, **kw):
        return self.forward_step(data_list, iteration, is_eval=True)
