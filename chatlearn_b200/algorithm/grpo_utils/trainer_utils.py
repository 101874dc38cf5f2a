"""Batch preparation for the policy trainer.

Parity: chatlearn/algorithm/grpo_utils/trainer_utils.py:27-194 and the
``preprocess_data_list`` part of policy_trainer.py:80-172.  The reference pads a
micro-batch to ``[B, S]``, builds masks and position ids, then un-pads into one
packed row for flash-attention varlen.  Here a micro-batch is built *directly*
as a packed row (tokens, positions, labels, loss mask, segment ids, per-token
old/ref log-probs and advantages), which is what the varlen kernels consume;
padded views are only produced on request (``pad_rows``).
"""
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from chatlearn_b200.utils import xfer


def split_microbatch(data_list: List[Dict], micro_batch_size: Optional[int] = None,
                     packing: bool = False, max_train_token: int = 0, max_reduce=None,
                     offset: int = 0) -> List[List[Dict]]:
    """Fixed-size micro-batches, or token-budget bins when ``packing``."""
    if packing:
        from .packing_utils import regroup_data_packing
        return regroup_data_packing(data_list, max_reduce, max_train_token, offset)
    assert micro_batch_size and micro_batch_size > 0
    out = []
    for s in range(0, len(data_list), micro_batch_size):
        mb = data_list[s:s + micro_batch_size]
        for j, d in enumerate(mb):
            d["id_in_list"] = s + j + offset
        out.append(mb)
    return out


@dataclass
class PackedBatch:
    tokens: torch.Tensor        # [T] int64
    positions: torch.Tensor     # [T] int64, restart at 0 per sequence
    labels: torch.Tensor        # [T] next token (last position of a sequence: 0, masked)
    loss_mask: torch.Tensor     # [T] float: 1 where the *label* is a response token
    seq_ids: torch.Tensor       # [T] int64 sequence index inside the micro-batch
    cu_seqlens: torch.Tensor    # [B+1] int32
    seq_lens: List[int]
    max_seqlen: int
    sample_ids: List[int]
    old_logprobs: Optional[torch.Tensor] = None   # [T] aligned with labels
    ref_logprobs: Optional[torch.Tensor] = None
    advantages: Optional[torch.Tensor] = None     # [T] (sequence advantage broadcast, or per token)
    values: Optional[torch.Tensor] = None         # [T] value estimates at rollout time (PPO critic)
    returns: Optional[torch.Tensor] = None        # [T] value targets
    pad: int = 0                                  # trailing pad tokens (SP/CP alignment)
    valid: Optional[torch.Tensor] = None          # [T] bool: a token of a sample (not alignment padding)
    mm: Any = None                                # per sample (pixel_values, image_grid_thw, visual_time_steps) or None (vision-language)

    def to(self, device):
        for k, v in vars(self).items():
            if isinstance(v, torch.Tensor):
                setattr(self, k, xfer.to_device(v, device, f"batch.{k}"))
        return self

    @property
    def num_tokens(self):
        return int(self.tokens.shape[0])


def _per_token(values, prompt_len: int, total_len: int):
    """Place per-response-token values (length = response length, or total-1) on the
    label grid of a sequence: index t holds the value for predicting token t+1."""
    out = torch.zeros(total_len, dtype=torch.float32)
    v = torch.as_tensor(values, dtype=torch.float32).flatten()
    resp = total_len - prompt_len
    if v.numel() == total_len - 1:
        out[:total_len - 1] = v
    elif v.numel() == total_len:          # value stored at the token it scores
        out[:total_len - 1] = v[1:]
    else:
        n = min(resp, v.numel())
        out[prompt_len - 1:prompt_len - 1 + n] = v[:n]
    return out


def pack_samples(samples: List[Dict[str, Any]], pad_multiple: int = 1, seq_multiple: int = 1,
                 pad_token: int = 0) -> PackedBatch:
    """Concatenate samples into one packed row.

    ``seq_multiple`` pads every sequence (context parallel needs multiples of
    ``2·cp``); ``pad_multiple`` pads the row (Ulysses needs a multiple of ``sp``).
    Padding tokens carry loss mask 0 and form their own attention segment."""
    toks, pos, lab, mask, sid, seq_lens, valid = [], [], [], [], [], [], []
    old, ref, adv = [], [], []
    have_old = all("old_logprobs" in s for s in samples)
    have_ref = all("ref_logprobs" in s for s in samples)
    have_adv = all("advantages" in s for s in samples)
    vals = [] if all("values" in s for s in samples) else None
    rets = [] if all("returns" in s for s in samples) else None
    for i, s in enumerate(samples):
        t = torch.as_tensor(s["all_tokens"], dtype=torch.long).flatten()
        pl, rl = int(s["prompt_token_length"]), int(s["response_token_length"])
        n = pl + rl
        t = t[:n]
        n_pad = (-n) % seq_multiple
        L = n + n_pad
        if n_pad:
            t = torch.cat([t, torch.full((n_pad,), pad_token, dtype=torch.long)])
        toks.append(t)
        pos.append(torch.arange(L))
        lb = torch.zeros(L, dtype=torch.long)
        lb[:n - 1] = t[1:n]
        lab.append(lb)
        m = torch.zeros(L, dtype=torch.float32)
        if "loss_mask" in s and s["loss_mask"] is not None:
            lm = torch.as_tensor(s["loss_mask"], dtype=torch.float32).flatten()[:n]
            m[:n - 1] = lm[1:n]                      # mask of the predicted token
        else:
            m[pl - 1:n - 1] = 1.0
        mask.append(m)
        sid.append(torch.full((L,), i, dtype=torch.long))
        valid.append(torch.arange(L) < n)
        seq_lens.append(L)
        if have_old:
            old.append(torch.nn.functional.pad(_per_token(s["old_logprobs"], pl, n), (0, n_pad)))
        if have_ref:
            ref.append(torch.nn.functional.pad(_per_token(s["ref_logprobs"], pl, n), (0, n_pad)))
        if have_adv:
            a = s["advantages"]
            if torch.is_tensor(a) and a.numel() > 1 or isinstance(a, (list, tuple)):
                # one advantage per response token (PPO with GAE)
                adv.append(torch.nn.functional.pad(_per_token(a, pl, n), (0, n_pad)))
            else:
                adv.append(torch.full((L,), float(a), dtype=torch.float32))
        for key, lst in (("values", vals), ("returns", rets)):
            if lst is not None:
                lst.append(torch.nn.functional.pad(_per_token(s[key], pl, n), (0, n_pad)))
    T = sum(seq_lens)
    pad = (-T) % pad_multiple
    if pad:
        toks.append(torch.full((pad,), pad_token, dtype=torch.long))
        pos.append(torch.arange(pad))
        lab.append(torch.zeros(pad, dtype=torch.long))
        mask.append(torch.zeros(pad))
        sid.append(torch.full((pad,), len(samples), dtype=torch.long))
        valid.append(torch.zeros(pad, dtype=torch.bool))
        seq_lens.append(pad)
        for lst in (old, ref, adv, vals, rets):
            if lst:
                lst.append(torch.zeros(pad))
    cu = torch.zeros(len(seq_lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(seq_lens, dtype=torch.int32).cumsum(0)
    cat = lambda xs: torch.cat(xs) if xs else None  # noqa: E731
    return PackedBatch(tokens=torch.cat(toks), positions=torch.cat(pos), labels=torch.cat(lab),
                       loss_mask=torch.cat(mask), seq_ids=torch.cat(sid), cu_seqlens=cu,
                       seq_lens=seq_lens, max_seqlen=max(seq_lens),
                       sample_ids=[int(s.get("id_in_list", i)) for i, s in enumerate(samples)],
                       old_logprobs=cat(old), ref_logprobs=cat(ref), advantages=cat(adv), values=cat(vals or []), returns=cat(rets or []), pad=pad, valid=torch.cat(valid) if valid else None,
                       mm=[(s.get("pixel_values"), s.get("image_grid_thw"), s.get("visual_time_steps")) for s in samples]
                       if any(s.get("pixel_values") is not None for s in samples) else None)


def unpack_per_sample(values: torch.Tensor, batch: PackedBatch, samples: List[Dict]) -> List[torch.Tensor]:
    """Cut a per-token vector of a packed row back into per-sample vectors of
    length ``total_len - 1`` (one value per predicted token)."""
    out, off = [], 0
    for i, s in enumerate(samples):
        n = int(s["prompt_token_length"]) + int(s["response_token_length"])
        out.append(values[off:off + n - 1].detach().float().cpu())
        off += batch.seq_lens[i]
    return out


def pad_rows(rows: List[torch.Tensor], pad_value=0, length: Optional[int] = None) -> torch.Tensor:
    """Right-pad 1-D tensors to a common length and stack."""
    L = length or max(int(r.shape[0]) for r in rows)
    out = rows[0].new_full((len(rows), L), pad_value)
    for i, r in enumerate(rows):
        out[i, :r.shape[0]] = r
    return out


def sp_split(x: torch.Tensor, sp_size: int, sp_rank: int, dim: int = 0) -> torch.Tensor:
    n = x.shape[dim] // sp_size
    return x.narrow(dim, sp_rank * n, n)
