"""Offline conversion of training checkpoints to HuggingFace safetensors (CPU only).

    python -m chatlearn_b200.offline_ckpt_converter --ckpt-dir <dir> --save-dir <out> \
        [--hf-dir <base model dir>] [--iter N] [--is-megatron]

Parity: chatlearn/offline_ckpt_converter.py:52-116, which merges the per-rank
FSDP ``.pt`` files (``model_world_size_{W}_rank_{R}.pt``) into HF safetensors using
the base model's index.  Both layouts written by this framework are handled:

* FSDP-style: every rank file holds its fp32 shard ``[lo, hi)`` of each flat
  parameter block; shards are concatenated, leaves cut out of the block and placed
  into HF tensors through the leaf layout of the architecture (``config.json``);
* Megatron-style: every ``mp_rank_*`` file carries its leaves *and* their HF
  rectangles, so the HF tensors are assembled by pasting rectangles.
"""
import argparse
import glob
import os
import re
from typing import Dict

import torch

from chatlearn_b200.checkpoint.safetensors_io import save_hf_checkpoint
from chatlearn_b200.models.nn import CausalLM, ModelArch


def convert_fsdp(ckpt_dir: str, arch: ModelArch, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    files = sorted(glob.glob(os.path.join(ckpt_dir, "model_world_size_*_rank_*.pt")),
                   key=lambda p: int(re.search(r"rank_(\d+)\.pt$", p).group(1)))
    assert files, f"no model_world_size_*_rank_*.pt under {ckpt_dir}"
    world = int(re.search(r"world_size_(\d+)_", files[0]).group(1))
    assert len(files) == world, f"expected {world} rank files, found {len(files)}"
    model = CausalLM(arch, dtype=torch.float32, device="cpu", pad_to=world)
    shards = [torch.load(f, weights_only=False, map_location="cpu") for f in files]
    for b in model.blocks:
        parts = sorted((s[b.name]["lo"], s[b.name]["shard"]) for s in shards)
        flat = torch.cat([p for _, p in parts]).float()
        assert flat.numel() == b.numel, f"block {b.name}: {flat.numel()} != {b.numel}"
        b.flat.copy_(flat)
    return model.hf_state_dict(dtype)


def convert_megatron(ckpt_dir: str, iteration=None, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    if iteration is None:
        with open(os.path.join(ckpt_dir, "latest_checkpointed_iteration.txt"), encoding="utf-8") as f:
            iteration = int(f.read().strip())
    out: Dict[str, torch.Tensor] = {}
    one_d = set()
    for f in sorted(glob.glob(os.path.join(ckpt_dir, f"iter_{iteration:07d}", "mp_rank_*", "model_optim_rng.pt"))):
        sd = torch.load(f, weights_only=False, map_location="cpu")
        for name, t in sd["model"].items():
            for hf_name, hf_shape, src, ext, dst, dst_index in sd["layout"][name]:
                full = out.setdefault(hf_name, torch.zeros(tuple(hf_shape), dtype=dtype))
                slab = t if t.dim() < 3 else t[dst_index]
                if t.dim() == 1:
                    one_d.add(hf_name)
                slab = slab.reshape(-1, slab.shape[-1]) if t.dim() > 1 else slab.reshape(-1, 1)
                full[src[0]:src[0] + ext[0], src[1]:src[1] + ext[1]] = \
                    slab[dst[0]:dst[0] + ext[0], dst[1]:dst[1] + ext[1]].to(dtype)
    for k in one_d:
        out[k] = out[k].squeeze(1)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt-dir", required=True)
    ap.add_argument("--save-dir", required=True)
    ap.add_argument("--hf-dir", default=None, help="directory with the base model's config.json (and tokenizer)")
    ap.add_argument("--iter", type=int, default=None)
    ap.add_argument("--is-megatron", action="store_true")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32", "fp16"])
    a = ap.parse_args(argv)
    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[a.dtype]
    cfg_dir = a.hf_dir or (os.path.join(a.ckpt_dir, "huggingface") if os.path.isdir(
        os.path.join(a.ckpt_dir, "huggingface")) else a.ckpt_dir)
    arch = ModelArch.from_pretrained(cfg_dir)
    sd = convert_megatron(a.ckpt_dir, a.iter, dtype) if a.is_megatron else convert_fsdp(a.ckpt_dir, arch, dtype)
    holder = CausalLM(arch, dtype=dtype, device="cpu", allocate=False)
    save_hf_checkpoint(holder, a.save_dir, dtype=dtype, state_dict=sd)
    if a.hf_dir:
        import shutil
        for fn in os.listdir(a.hf_dir):
            if fn.startswith("tokenizer") or fn in ("vocab.json", "merges.txt", "special_tokens_map.json",
                                                     "generation_config.json"):
                shutil.copy(os.path.join(a.hf_dir, fn), os.path.join(a.save_dir, fn))
    print(f"wrote {len(sd)} tensors to {a.save_dir}")


if __name__ == "__main__":
    main()
