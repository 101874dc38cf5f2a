"""Sequence packing (dynamic batching) for training micro-batches.

Parity: chatlearn/algorithm/grpo_utils/packing_utils.py:23-148.  Same two-pass
scheme: best-fit-decreasing into bins of capacity ``max_train_token`` (a
sequence fits only if the remaining space is strictly larger than its length),
the bin count is MAX-reduced over the ranks that must run in lock step, then the
sequences are re-balanced into exactly that many bins (longest first, always
into the lightest bin) and bins are ordered by load, heaviest first.  The
implementation keeps running bin loads instead of re-summing lists.
"""
import warnings
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple


def bin_packing(seq_len_list: Sequence[int], max_train_token: int) -> Tuple[List[List[int]], List[List[int]]]:
    if any(n > max_train_token for n in seq_len_list):
        warnings.warn(f"a sequence of {max(seq_len_list)} tokens exceeds max_token_in_packing="
                      f"{max_train_token}; it gets a bin of its own")
    order = sorted(range(len(seq_len_list)), key=lambda i: seq_len_list[i], reverse=True)
    ids: List[List[int]] = []
    lens: List[List[int]] = []
    load: List[int] = []
    for i in order:
        n = seq_len_list[i]
        best, best_space = None, None
        for b, used in enumerate(load):
            space = max_train_token - used
            if space > n and (best_space is None or space < best_space):
                best, best_space = b, space
        if best is None:
            ids.append([i]); lens.append([n]); load.append(n)
        else:
            ids[best].append(i); lens[best].append(n); load[best] += n
    return ids, lens


def bin_packing_fix_bin(seq_len_list: Sequence[int], bin_size: int) -> Tuple[List[List[int]], List[List[int]]]:
    order = sorted(range(len(seq_len_list)), key=lambda i: seq_len_list[i], reverse=True)
    ids = [[] for _ in range(bin_size)]
    lens = [[] for _ in range(bin_size)]
    load = [0] * bin_size
    for i in order:
        b = min(range(bin_size), key=lambda j: load[j])   # first lightest bin
        ids[b].append(i); lens[b].append(seq_len_list[i]); load[b] += seq_len_list[i]
    rank = sorted(range(bin_size), key=lambda j: (load[j], ids[j]), reverse=True)
    return [ids[j] for j in rank], [lens[j] for j in rank]


def regroup_data_packing(data_list: List[Dict[str, Any]], max_reduce: Optional[Callable[[int], int]],
                         max_train_token: int, offset: int = 0) -> List[List[Dict[str, Any]]]:
    """Split samples into micro-batches of at most ``max_train_token`` tokens.

    ``max_reduce(n)`` returns the maximum of ``n`` over all ranks that must run the
    same number of micro-batches (``None`` → single rank)."""
    total = [int(d["prompt_token_length"]) + int(d["response_token_length"]) for d in data_list]
    bins, _ = bin_packing(total, max_train_token)
    n_bins = len(bins)
    if max_reduce is not None:
        n_bins = int(max_reduce(n_bins))
    bins, _ = bin_packing_fix_bin(total, max(n_bins, 1))
    out = []
    for ids in bins:
        mb = []
        for i in ids:
            s = data_list[i]
            s["id_in_list"] = i + offset
            mb.append(s)
        out.append(mb)
    return out
