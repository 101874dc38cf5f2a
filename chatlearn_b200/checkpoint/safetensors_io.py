"""HuggingFace safetensors reading and writing with direct sharded reads.

The reference loads HF checkpoints by having every rank read whole files into a
3 G-element zero bucket that is then all-reduced and re-distributed
(chatlearn/models/fsdp_module.py:103-186), and saves through
``save_pretrained`` (:577-621).  The safetensors container is simple — an 8-byte
little-endian header length, a JSON header ``{name: {dtype, shape, data_offsets}}``
and raw little-endian data — so here each rank memory-maps the files and copies
only the rectangles its own leaves need; no collective, no staging bucket.  The
writer emits the same container plus ``model.safetensors.index.json`` and
``config.json``, so the output loads in ``transformers``.
"""
import json
import mmap
import os
import struct
from typing import Dict, List, Optional

import torch

_DTYPES = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64,
           "I32": torch.int32, "U8": torch.uint8, "I8": torch.int8, "BOOL": torch.bool,
           "F64": torch.float64, "I16": torch.int16}
_NAMES = {v: k for k, v in _DTYPES.items()}


def has_safetensors(path: str) -> bool:
    return bool(path) and os.path.isdir(path) and any(f.endswith(".safetensors") for f in os.listdir(path))


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        self.header = json.loads(self._f.read(n))
        self.meta = self.header.pop("__metadata__", {})
        self.base = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def keys(self):
        return self.header.keys()

    def tensor(self, name: str) -> torch.Tensor:
        """Zero-copy view of a tensor (read-only memory map)."""
        info = self.header[name]
        dt = _DTYPES[info["dtype"]]
        s, e = info["data_offsets"]
        buf = memoryview(self._mm)[self.base + s:self.base + e]
        t = torch.frombuffer(buf, dtype=dt) if e > s else torch.empty(0, dtype=dt)
        return t.view(info["shape"])

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass  # views of the map are still alive; the OS unmaps at exit
        self._f.close()


class SafetensorsDir:
    """All ``*.safetensors`` of a HF directory behind one name → tensor lookup."""

    def __init__(self, path: str):
        self.path = path
        self.files: Dict[str, SafetensorsFile] = {}
        self.where: Dict[str, str] = {}
        idx = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx, "r", encoding="utf-8") as f:
                self.where = dict(json.load(f)["weight_map"])
        else:
            for fn in sorted(os.listdir(path)):
                if fn.endswith(".safetensors"):
                    sf = self._open(fn)
                    for k in sf.keys():
                        self.where[k] = fn

    def _open(self, fn: str) -> SafetensorsFile:
        if fn not in self.files:
            self.files[fn] = SafetensorsFile(os.path.join(self.path, fn))
        return self.files[fn]

    def __contains__(self, name):
        return name in self.where

    def get(self, name: str) -> Optional[torch.Tensor]:
        fn = self.where.get(name)
        return self._open(fn).tensor(name) if fn else None

    def keys(self):
        return self.where.keys()

    def close(self):
        for f in self.files.values():
            f.close()


@torch.no_grad()
def load_into_model(model, path: str, strict: bool = True) -> List[str]:
    """Fill a (possibly TP/EP-sharded) ``CausalLM`` from a HF directory, reading only
    the rectangles each leaf needs."""
    d = SafetensorsDir(path)
    missing = []
    for _, p, lf, _ in model.named_leaves():
        for s in lf.segments:
            src = d.get(s.hf_name)
            if src is None and s.hf_name == "lm_head.weight":
                src = d.get("model.embed_tokens.weight")     # tied checkpoints
            if src is None:
                missing.append(s.hf_name)
                continue
            src = src.reshape(s.hf_shape)
            slab = p if len(lf.shape) < 3 else p[s.dst_index]
            slab = slab.view(lf.matrix_shape)
            r0, c0 = s.dst_start
            rs, cs = s.src_start
            nr, nc = s.extent
            slab[r0:r0 + nr, c0:c0 + nc].copy_(src[rs:rs + nr, cs:cs + nc])
    d.close()
    if strict and missing:
        raise KeyError(f"tensors missing from {path}: {sorted(set(missing))[:8]}")
    return missing


def write_safetensors(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict] = None):
    header, off = {}, 0
    order = list(tensors)
    for k in order:
        t = tensors[k]
        n = t.numel() * t.element_size()
        header[k] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    if metadata:
        header["__metadata__"] = {str(a): str(b) for a, b in metadata.items()}
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for k in order:
            t = tensors[k].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def save_hf_checkpoint(model, path: str, dtype=torch.bfloat16, max_shard_bytes: int = 5 << 30,
                       state_dict: Optional[Dict[str, torch.Tensor]] = None):
    """Write ``config.json`` + sharded safetensors + index for a complete model."""
    os.makedirs(path, exist_ok=True)
    sd = state_dict if state_dict is not None else model.hf_state_dict(dtype)
    model.arch.save_pretrained(path)
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for k, v in sd.items():
        n = v.numel() * v.element_size()
        if size and size + n > max_shard_bytes:
            shards.append({})
            size = 0
        shards[-1][k] = v.to(dtype) if v.is_floating_point() else v
        size += n
    weight_map, total = {}, 0
    for i, sh in enumerate(shards):
        fn = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        write_safetensors(sh, os.path.join(path, fn), {"format": "pt"})
        for k, v in sh.items():
            weight_map[k] = fn
            total += v.numel() * v.element_size()
    with open(os.path.join(path, "model.safetensors.index.json"), "w", encoding="utf-8") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
