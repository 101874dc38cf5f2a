"""Offline check of a trainer → rollout parameter sync.

Parity: chatlearn/tools/check_parameter_sync.py (compare dumped tensors, print
``PASS|…`` / ``DIFF|…`` / ``NOT_EXISTS|…`` lines and totals).  With
``DEBUG_SYNC_PARAMETERS_PATH=<dir>`` set, the engine dumps after the first sync

* ``<dir>/after_sync_parameter/<role>_rank<r>.pt`` – every rollout rank's leaves plus
  its architecture and tensor/expert-parallel coordinates,
* ``<dir>/trainer_hf/rank<r>.pt`` – every trainer rank's weights under their HF names
  (partial tensors when the trainer is model-parallel).

``python -m chatlearn_b200.synchronizer.check_parameter_sync --root_dir <dir>`` merges
the trainer dumps into whole HF tensors, loads them into a model with each rollout
rank's coordinates, and compares leaf by leaf.
"""
import argparse
import glob
import os
from typing import Dict

import torch


def dump_expected(src, path: str):
    if not src.is_member or getattr(src, "model", None) is None:
        return
    os.makedirs(path, exist_ok=True)
    sd = {k: v.detach().float().cpu() for k, v in src.model.hf_state_dict().items()}
    torch.save(sd, os.path.join(path, f"rank{src.get_rank()}.pt"))


def merge_partials(paths) -> Dict[str, torch.Tensor]:
    """Model-parallel ranks hold disjoint (or identical, when replicated) pieces of every
    HF tensor, zero elsewhere: fill the holes of the running result."""
    full: Dict[str, torch.Tensor] = {}
    for p in sorted(paths):
        for k, v in torch.load(p, map_location="cpu").items():
            if k not in full:
                full[k] = v.clone()
            else:
                full[k] = torch.where(full[k] == 0, v, full[k])
    return full


def compare(root_dir: str, rtol: float = 0.0, atol: float = 0.0, verbose: bool = True):
    from chatlearn_b200.models.nn import CausalLM
    from chatlearn_b200.models.nn.arch import ModelArch
    hf = merge_partials(glob.glob(os.path.join(root_dir, "trainer_hf", "rank*.pt")))
    total = diff = missing = 0
    for f in sorted(glob.glob(os.path.join(root_dir, "after_sync_parameter", "*.pt"))):
        d = torch.load(f, map_location="cpu")
        arch = ModelArch(**d["arch"])
        want = CausalLM(arch, dtype=torch.float32, device="cpu", tp=d["tp"], tp_rank=d["tp_rank"], ep=d["ep"],
                        ep_rank=d["ep_rank"])
        want.load_hf_state_dict(hf, strict=False)
        expected = {n: p for n, p, _, _ in want.named_leaves()}
        tag = os.path.basename(f)[:-3]
        for name, got in d["leaves"].items():
            total += 1
            msg = f"{tag}|{name}"
            if name not in expected:
                missing += 1
                print(f"NOT_EXISTS|{msg}|NOT_EXISTS", flush=True)
                continue
            exp = expected[name]
            if got.shape != exp.shape or not torch.allclose(got, exp, rtol=rtol, atol=atol):
                diff += 1
                print(f"DIFF|{msg}|{tuple(got.shape)}|{got.mean():.6g}|{tuple(exp.shape)}|{exp.mean():.6g}", flush=True)
            elif verbose:
                print(f"PASS|{msg}")
    print(f"ALL: {total}, DIFF: {diff}, NOT_EXISTS: {missing}")
    return total, diff, missing


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--root_dir", type=str, required=True, help="directory of the dumped parameters")
    ap.add_argument("--quiet", action="store_true")
    a = ap.parse_args()
    _, d, m = compare(a.root_dir, verbose=not a.quiet)
    raise SystemExit(1 if d or m else 0)
