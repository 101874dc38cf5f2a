"""geo3k reward: 0.9 · accuracy + 0.1 · format
(chatlearn/utils/rule_reward_score/geo3k.py:8-25): the response must be
``<think>…</think>`` followed by a ``\\boxed{}`` answer."""
import re

from .math import is_equiv, last_boxed_only_string, remove_boxed

_FMT = re.compile(r"<think>.*</think>.*\\boxed\{.*\}.*", re.S)


def format_reward(text: str) -> float:
    return 1.0 if _FMT.fullmatch(text) else 0.0


def acc_reward(text: str, ground_truth: str) -> float:
    boxed = last_boxed_only_string(text)
    if boxed is None:
        return 0.0
    return 1.0 if is_equiv(remove_boxed(boxed), ground_truth) else 0.0


def compute_score(text: str, ground_truth: str, format_score: float = 0.1) -> float:
    return (1.0 - format_score) * acc_reward(text, ground_truth) + format_score * format_reward(text)
