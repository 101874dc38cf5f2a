"""Synthetic prompts and rule rewards for offline benchmarks and tests.

Prompts are uniform-random token ids with lengths uniform in ``[lo, hi]``,
generated from a seed, in the dataset record format the prompt pipeline reads
(``input_ids`` + ``reward_model.ground_truth``).
"""
import json
from typing import Dict, List

import torch


def make_prompts(num: int, lo: int, hi: int, vocab_size: int, seed: int = 0,
                 data_source: str = "synthetic", reserved_top: int = 1) -> List[Dict]:
    """``reserved_top`` ids at the top of the vocabulary (EOS etc.) are never drawn."""
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (num,), generator=g).tolist()
    out = []
    for n in lens:
        ids = torch.randint(0, vocab_size - reserved_top, (n,), generator=g).tolist()
        out.append({"data_source": data_source, "input_ids": ids,
                    "reward_model": {"ground_truth": ""}})
    return out


def write_jsonl(rows: List[Dict], path: str):
    with open(path, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")


def reward_last_token_mod7(response_ids) -> float:
    """1.0 if the last generated token id is a multiple of 7."""
    if len(response_ids) == 0:
        return 0.0
    return 1.0 if int(response_ids[-1]) % 7 == 0 else 0.0


def reward_hash_p30(response_ids) -> float:
    """Deterministic hash of the response ids into {0,1} with P(1) ≈ 0.3
    (FNV-1a over the ids, accepted when the hash falls in the low 30 %)."""
    h = 0xcbf29ce484222325
    for t in response_ids:
        h ^= int(t) & 0xFFFFFFFF
        h = (h * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    return 1.0 if (h % 1000) < 300 else 0.0


SYNTHETIC_REWARDS = {"mod7": reward_last_token_mod7, "hash30": reward_hash_p30}
