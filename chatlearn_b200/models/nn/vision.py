"""Vision tower and multimodal position logic of Qwen2.5-VL-style models.

Parity: what the reference gets from HuggingFace through
chatlearn/models/patches/transformers/qwen2_5_vl_patch.py (vision tower, mrope) and
chatlearn/data/vision_utils.py (grids).  Written against the published architecture:

* patches ``[N, C·Tp·P·P]`` → linear patch embedding;
* 2-D rotary position per patch (row and column frequencies side by side), patches stored in
  spatial-merge blocks;
* transformer blocks (RMSNorm, fused QKV with bias, SwiGLU MLP with bias); most blocks attend
  inside windows, the ``fullatt_block_indexes`` ones over the whole image — both are packed
  variable-length attention over different ``cu_seqlens``, after the merge-block groups are
  re-ordered window by window;
* patch merger: RMSNorm, concatenate each block of ``merge²`` patches, two-layer GELU MLP to the
  language model's width; the window order is undone at the end.

Weights live in a dict keyed by the HuggingFace names (``visual.…``), so checkpoints load by name.
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from chatlearn_b200 import ops


@dataclass
class VisionArch:
    depth: int = 32
    hidden_size: int = 1280
    intermediate_size: int = 3420
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 3584
    window_size: int = 112
    fullatt_block_indexes: List[int] = field(default_factory=lambda: [7, 15, 23, 31])
    rms_norm_eps: float = 1e-6

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size

    @property
    def merge_unit(self) -> int:
        return self.spatial_merge_size ** 2

    @classmethod
    def from_hf_dict(cls, d: Dict) -> "VisionArch":
        keys = {f for f in cls.__dataclass_fields__}
        kw = {k: v for k, v in d.items() if k in keys}
        if "in_chans" in d:
            kw["in_channels"] = d["in_chans"]
        return cls(**kw)


def vision_param_shapes(a: VisionArch) -> Dict[str, Tuple[int, ...]]:
    H, I = a.hidden_size, a.intermediate_size
    out = {"visual.patch_embed.proj.weight": (H, a.patch_dim)}
    for i in range(a.depth):
        b = f"visual.blocks.{i}."
        out.update({b + "norm1.weight": (H,), b + "norm2.weight": (H,),
                    b + "attn.qkv.weight": (3 * H, H), b + "attn.qkv.bias": (3 * H,),
                    b + "attn.proj.weight": (H, H), b + "attn.proj.bias": (H,),
                    b + "mlp.gate_proj.weight": (I, H), b + "mlp.gate_proj.bias": (I,),
                    b + "mlp.up_proj.weight": (I, H), b + "mlp.up_proj.bias": (I,),
                    b + "mlp.down_proj.weight": (H, I), b + "mlp.down_proj.bias": (H,)})
    M = H * a.merge_unit
    out.update({"visual.merger.ln_q.weight": (H,), "visual.merger.mlp.0.weight": (M, M), "visual.merger.mlp.0.bias": (M,),
                "visual.merger.mlp.2.weight": (a.out_hidden_size, M), "visual.merger.mlp.2.bias": (a.out_hidden_size,)})
    return out


def patch_positions(grid_thw: Sequence[Sequence[int]], merge: int) -> torch.Tensor:
    """(row, column) of every patch in storage order: merge blocks are contiguous."""
    out = []
    for t, h, w in grid_thw:
        rows = torch.arange(h).view(h // merge, merge, 1, 1).expand(h // merge, merge, w // merge, merge)
        cols = torch.arange(w).view(1, 1, w // merge, merge).expand(h // merge, merge, w // merge, merge)
        rc = torch.stack([rows.permute(0, 2, 1, 3).reshape(-1), cols.permute(0, 2, 1, 3).reshape(-1)], -1)
        out.append(rc.repeat(t, 1))
    return torch.cat(out, 0)


def window_order(grid_thw: Sequence[Sequence[int]], a: VisionArch) -> Tuple[torch.Tensor, List[int]]:
    """Order of the merge-block groups window by window, and the cumulative patch counts of the
    windows (empty windows removed)."""
    m = a.spatial_merge_size
    win = a.window_size // m // a.patch_size
    order, cu, base = [], [0], 0
    for t, h, w in grid_thw:
        gh, gw = h // m, w // m
        idx = torch.arange(t * gh * gw).view(t, gh, gw)
        ph, pw = win - gh % win, win - gw % win            # (a full extra window of padding when already aligned)
        idx = F.pad(idx, (0, pw, 0, ph), value=-1)
        nh, nw = (gh + ph) // win, (gw + pw) // win
        idx = idx.view(t, nh, win, nw, win).permute(0, 1, 3, 2, 4).reshape(t * nh * nw, win * win)
        counts = (idx >= 0).sum(1)
        order.append(idx.reshape(-1)[idx.reshape(-1) >= 0] + base)
        for c in counts.tolist():
            if c:
                cu.append(cu[-1] + c * a.merge_unit)
        base += t * gh * gw
    return torch.cat(order), cu


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), -1)


class VisionTower:
    def __init__(self, arch: VisionArch, dtype=torch.float32, device="cpu"):
        self.arch, self.dtype, self.device = arch, dtype, torch.device(device)
        self.params: Dict[str, torch.Tensor] = {
            k: torch.zeros(s, dtype=dtype, device=self.device) for k, s in vision_param_shapes(arch).items()}

    def init_weights(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator().manual_seed(seed)
        for k, p in self.params.items():
            if k.endswith("norm1.weight") or k.endswith("norm2.weight") or k.endswith("ln_q.weight"):
                p.fill_(1.0)
            elif k.endswith(".bias"):
                p.zero_()
            else:
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
        return self

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True) -> List[str]:
        """Accepts ``visual.*`` or ``model.visual.*`` names; the patch-embedding convolution kernel is
        flattened to a matrix."""
        missing = []
        for k, p in self.params.items():
            src = sd.get(k, sd.get("model." + k))
            if src is None:
                missing.append(k)
                continue
            p.copy_(src.reshape(p.shape).to(p.dtype))
        if strict and missing:
            raise KeyError(f"vision weights missing: {missing[:4]} ...")
        return missing

    def hf_state_dict(self) -> Dict[str, torch.Tensor]:
        a = self.arch
        out = dict(self.params)
        out["visual.patch_embed.proj.weight"] = self.params["visual.patch_embed.proj.weight"].view(
            a.hidden_size, a.in_channels, a.temporal_patch_size, a.patch_size, a.patch_size)
        return out

    def _lin(self, x, name):
        return ops.linear(x, self.params[name + ".weight"], self.params.get(name + ".bias"))

    def forward(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        """``pixel_values [N, patch_dim]``, ``grid_thw`` = (t, h, w) per image in patches.  Returns the
        merged image embeddings ``[N / merge², out_hidden]`` in the order of the input patches."""
        a, P = self.arch, self.params
        grid = [tuple(int(v) for v in g) for g in (grid_thw.tolist() if torch.is_tensor(grid_thw) else grid_thw)]
        x = ops.linear(pixel_values.to(self.dtype), P["visual.patch_embed.proj.weight"])
        N, H, nh = x.shape[0], a.hidden_size, a.num_heads
        d = H // nh
        # rotary table: row frequencies then column frequencies, each d/4 wide
        rc = patch_positions(grid, a.spatial_merge_size).to(x.device)
        inv = 1.0 / (10000.0 ** (torch.arange(0, d // 2, 2, dtype=torch.float32, device=x.device) / (d // 2)))
        ang = torch.cat([rc[:, :1].float() * inv, rc[:, 1:].float() * inv], -1)          # [N, d/2]
        order, cu_win = window_order(grid, a)
        order = order.to(x.device)
        u = a.merge_unit
        x = x.view(N // u, u, H)[order].reshape(N, H)
        ang = ang.view(N // u, u, -1)[order].reshape(N, -1)
        emb = torch.cat([ang, ang], -1)
        cos, sin = emb.cos()[:, None, :], emb.sin()[:, None, :]
        cu_full = [0]
        for t, h, w in grid:
            for _ in range(t):
                cu_full.append(cu_full[-1] + h * w)
        cu_full_t = torch.tensor(cu_full, dtype=torch.int32, device=x.device)
        cu_win_t = torch.tensor(cu_win, dtype=torch.int32, device=x.device)
        scale = d ** -0.5
        for i in range(a.depth):
            b = f"visual.blocks.{i}."
            h_ = ops.rmsnorm(x, P[b + "norm1.weight"], a.rms_norm_eps)
            qkv = self._lin(h_, b + "attn.qkv").view(N, 3, nh, d)
            q, k, v = qkv[:, 0].float(), qkv[:, 1].float(), qkv[:, 2]
            q = (q * cos + _rotate_half(q) * sin).to(x.dtype)
            k = (k * cos + _rotate_half(k) * sin).to(x.dtype)
            full = i in a.fullatt_block_indexes
            cu = cu_full_t if full else cu_win_t
            lens = (cu[1:] - cu[:-1])
            o = ops.attention_varlen(q.contiguous(), k.contiguous(), v.contiguous(), cu, int(lens.max()), scale, False)
            x = x + self._lin(o.reshape(N, H), b + "attn.proj")
            h_ = ops.rmsnorm(x, P[b + "norm2.weight"], a.rms_norm_eps)
            g_ = F.silu(self._lin(h_, b + "mlp.gate_proj")) * self._lin(h_, b + "mlp.up_proj")
            x = x + self._lin(g_, b + "mlp.down_proj")
        x = ops.rmsnorm(x, P["visual.merger.ln_q.weight"], a.rms_norm_eps).view(N // u, u * H)
        x = self._lin(F.gelu(self._lin(x, "visual.merger.mlp.0")), "visual.merger.mlp.2")
        return x[torch.argsort(order)]

    __call__ = forward


# ---------------------------------------------------------------------------------------------
# Qwen3-VL: learned position table (bilinear interpolation to the image grid), LayerNorm blocks with
# a GELU MLP, attention over whole frames (no windows), and "deep-stack" taps: the outputs of a few
# blocks go through their own mergers and are added to the language model's early hidden states.
# ---------------------------------------------------------------------------------------------
@dataclass
class Vision3Arch:
    depth: int = 27
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 4096
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: List[int] = field(default_factory=lambda: [8, 16, 24])
    hidden_act: str = "gelu_pytorch_tanh"

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size

    @property
    def merge_unit(self) -> int:
        return self.spatial_merge_size ** 2

    @classmethod
    def from_hf_dict(cls, d: Dict) -> "Vision3Arch":
        keys = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in keys})


def vision3_param_shapes(a: Vision3Arch) -> Dict[str, Tuple[int, ...]]:
    H, I, M = a.hidden_size, a.intermediate_size, a.hidden_size * a.merge_unit
    out = {"visual.patch_embed.proj.weight": (H, a.patch_dim), "visual.patch_embed.proj.bias": (H,),
           "visual.pos_embed.weight": (a.num_position_embeddings, H)}
    for i in range(a.depth):
        b = f"visual.blocks.{i}."
        out.update({b + "norm1.weight": (H,), b + "norm1.bias": (H,), b + "norm2.weight": (H,), b + "norm2.bias": (H,),
                    b + "attn.qkv.weight": (3 * H, H), b + "attn.qkv.bias": (3 * H,),
                    b + "attn.proj.weight": (H, H), b + "attn.proj.bias": (H,),
                    b + "mlp.linear_fc1.weight": (I, H), b + "mlp.linear_fc1.bias": (I,),
                    b + "mlp.linear_fc2.weight": (H, I), b + "mlp.linear_fc2.bias": (H,)})

    def merger(prefix, norm_dim):
        out.update({prefix + "norm.weight": (norm_dim,), prefix + "norm.bias": (norm_dim,),
                    prefix + "linear_fc1.weight": (M, M), prefix + "linear_fc1.bias": (M,),
                    prefix + "linear_fc2.weight": (a.out_hidden_size, M), prefix + "linear_fc2.bias": (a.out_hidden_size,)})
    merger("visual.merger.", H)
    for j in range(len(a.deepstack_visual_indexes)):
        merger(f"visual.deepstack_merger_list.{j}.", M)
    return out


class VisionTower3(VisionTower):
    """Returns ``(image embeddings, [deep-stack features per tap])``, all ``[N / merge², out_hidden]``."""

    def __init__(self, arch: Vision3Arch, dtype=torch.float32, device="cpu"):  # pylint: disable=super-init-not-called
        self.arch, self.dtype, self.device = arch, dtype, torch.device(device)
        self.params = {k: torch.zeros(s, dtype=dtype, device=self.device) for k, s in vision3_param_shapes(arch).items()}

    def init_weights(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator().manual_seed(seed)
        for k, p in self.params.items():
            if ".norm" in k and k.endswith(".weight"):
                p.fill_(1.0)
            elif k.endswith(".bias"):
                p.zero_()
            else:
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
        return self

    def hf_state_dict(self):
        a = self.arch
        out = dict(self.params)
        out["visual.patch_embed.proj.weight"] = self.params["visual.patch_embed.proj.weight"].view(
            a.hidden_size, a.in_channels, a.temporal_patch_size, a.patch_size, a.patch_size)
        return out

    def _pos_table(self, grid) -> torch.Tensor:
        """Learned position embedding of every patch: the square table is sampled bilinearly at the
        image's own grid, then put into merge-block order."""
        a = self.arch
        side = int(round(a.num_position_embeddings ** 0.5))
        table = self.params["visual.pos_embed.weight"].float()
        out, m = [], a.spatial_merge_size
        for t, h, w in grid:
            ys, xs = torch.linspace(0, side - 1, h, device=table.device), torch.linspace(0, side - 1, w, device=table.device)
            y0, x0 = ys.long(), xs.long()
            y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
            dy, dx = (ys - y0)[:, None, None], (xs - x0)[None, :, None]
            e = lambda yy, xx: table[(yy[:, None] * side + xx[None, :])]          # noqa: E731  [h, w, H]
            pe = e(y0, x0) * (1 - dy) * (1 - dx) + e(y0, x1) * (1 - dy) * dx + e(y1, x0) * dy * (1 - dx) + e(y1, x1) * dy * dx
            pe = pe.view(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            out.append(pe.repeat(t, 1))
        return torch.cat(out, 0)

    def _merge(self, x, prefix, post_norm: bool):
        a, P = self.arch, self.params
        M = a.hidden_size * a.merge_unit
        if post_norm:
            x = F.layer_norm(x.view(-1, M), (M,), P[prefix + "norm.weight"], P[prefix + "norm.bias"], 1e-6)
        else:
            x = F.layer_norm(x, (a.hidden_size,), P[prefix + "norm.weight"], P[prefix + "norm.bias"], 1e-6).view(-1, M)
        return self._lin(F.gelu(self._lin(x, prefix + "linear_fc1")), prefix + "linear_fc2")

    def forward(self, pixel_values: torch.Tensor, grid_thw):
        a, P = self.arch, self.params
        grid = [tuple(int(v) for v in g) for g in (grid_thw.tolist() if torch.is_tensor(grid_thw) else grid_thw)]
        x = ops.linear(pixel_values.to(self.dtype), P["visual.patch_embed.proj.weight"], P["visual.patch_embed.proj.bias"])
        x = x + self._pos_table(grid).to(x.dtype)
        N, H, nh = x.shape[0], a.hidden_size, a.num_heads
        d = H // nh
        rc = patch_positions(grid, a.spatial_merge_size).to(x.device)
        inv = 1.0 / (10000.0 ** (torch.arange(0, d // 2, 2, dtype=torch.float32, device=x.device) / (d // 2)))
        ang = torch.cat([rc[:, :1].float() * inv, rc[:, 1:].float() * inv], -1)
        emb = torch.cat([ang, ang], -1)
        cos, sin = emb.cos()[:, None, :], emb.sin()[:, None, :]
        cu = [0]
        for t, h, w in grid:
            for _ in range(t):
                cu.append(cu[-1] + h * w)
        cu_t = torch.tensor(cu, dtype=torch.int32, device=x.device)
        max_len = max(h * w for _, h, w in grid)
        act = (lambda z: F.gelu(z, approximate="tanh")) if "tanh" in a.hidden_act else F.gelu
        taps = []
        for i in range(a.depth):
            b = f"visual.blocks.{i}."
            h_ = F.layer_norm(x, (H,), P[b + "norm1.weight"], P[b + "norm1.bias"], 1e-6)
            qkv = self._lin(h_, b + "attn.qkv").view(N, 3, nh, d)
            q, k, v = qkv[:, 0].float(), qkv[:, 1].float(), qkv[:, 2]
            q = (q * cos + _rotate_half(q) * sin).to(x.dtype)
            k = (k * cos + _rotate_half(k) * sin).to(x.dtype)
            o = ops.attention_varlen(q.contiguous(), k.contiguous(), v.contiguous(), cu_t, max_len, d ** -0.5, False)
            x = x + self._lin(o.reshape(N, H), b + "attn.proj")
            h_ = F.layer_norm(x, (H,), P[b + "norm2.weight"], P[b + "norm2.bias"], 1e-6)
            x = x + self._lin(act(self._lin(h_, b + "mlp.linear_fc1")), b + "mlp.linear_fc2")
            if i in a.deepstack_visual_indexes:
                taps.append(self._merge(x, f"visual.deepstack_merger_list.{a.deepstack_visual_indexes.index(i)}.", True))
        return self._merge(x, "visual.merger.", False), taps

    __call__ = forward


def mrope_positions(input_ids: torch.Tensor, image_grid_thw, image_token_id: int, merge: int,
                    video_token_id: Optional[int] = None, time_steps=None) -> Tuple[torch.Tensor, int]:
    """Three-component (time, row, column) positions of one sequence and the offset that later text
    positions carry: text tokens count up with all components equal; an image or a video occupies a
    (t, h/merge, w/merge) grid starting at the current position, and the text after it continues one past the
    largest position of the grid.  ``image_grid_thw`` lists the grids of all images and videos in the order of
    their placeholder runs; ``time_steps[i]`` is the temporal position step between two frame groups of item ``i``
    (Qwen2.5-VL: seconds per temporal grid step x the tower's ``tokens_per_second``, truncated per frame group;
    ``None``: one position per frame group).  The reference patches the same rule into HuggingFace's model
    (chatlearn/models/patches/transformers/qwen2_5_vl_patch.py:10-140)."""
    ids = input_ids.tolist()
    grids = [tuple(int(v) for v in g) for g in (image_grid_thw.tolist() if torch.is_tensor(image_grid_thw) else (image_grid_thw or []))]
    visual = {t for t in (image_token_id, video_token_id) if t is not None}
    out, cur, i, gi = [], 0, 0, 0
    n = len(ids)
    while i < n:
        if ids[i] in visual and gi < len(grids):        # (a placeholder token the model generated itself is text)
            t, h, w = grids[gi]
            step = time_steps[gi] if time_steps is not None and time_steps[gi] is not None else 1
            gi += 1
            gh, gw = h // merge, w // merge
            cnt = t * gh * gw
            tt = (torch.arange(t) * step).long().view(t, 1, 1).expand(t, gh, gw).reshape(-1)
            hh = torch.arange(gh).view(1, gh, 1).expand(t, gh, gw).reshape(-1)
            ww = torch.arange(gw).view(1, 1, gw).expand(t, gh, gw).reshape(-1)
            out.append(torch.stack([tt, hh, ww]) + cur)
            cur += max(int(tt[-1]) + 1, gh, gw)
            i += cnt
        else:
            j = i + 1 if ids[i] in visual else i
            while j < n and (ids[j] not in visual or gi >= len(grids)):
                j += 1
            out.append((torch.arange(j - i) + cur).view(1, -1).expand(3, -1))
            cur += j - i
            i = j
    pos = torch.cat(out, 1) if out else torch.zeros(3, 0, dtype=torch.long)
    delta = int(pos.max().item()) + 1 - n if n else 0
    return pos.long(), delta


def build_vision_tower(arch, dtype, device, load: str = None, seed: int = 4321):
    """The (frozen) vision tower of a vision-language role, or ``None`` for text models.  Weights come
    from the HF checkpoint directory ``load`` when it holds them, else from a seeded random init (the
    same on every role, so trainer and rollout agree)."""
    if getattr(arch, "vision_config", None) is None:
        return None
    if "deepstack_visual_indexes" in arch.vision_config or "num_position_embeddings" in arch.vision_config:
        tower = VisionTower3(Vision3Arch.from_hf_dict(arch.vision_config), dtype=dtype, device=device)
    else:
        tower = VisionTower(VisionArch.from_hf_dict(arch.vision_config), dtype=dtype, device=device)
    loaded = False
    if load:
        from chatlearn_b200.checkpoint.safetensors_io import SafetensorsDir, has_safetensors
        if has_safetensors(load):
            d = SafetensorsDir(load)
            sd = {}
            for k in tower.params:
                t = d.get(k)
                if t is None:
                    t = d.get("model." + k)
                if t is not None:
                    sd[k] = t
            if sd:
                tower.load_hf_state_dict(sd, strict=True)
                loaded = True
            d.close()
    if not loaded:
        tower.init_weights(seed)
    return tower


def attach_vision_block(lm, tower, pad_to: int = 1):
    """Make the tower's weights a parameter block of the language model ("vision", after the head), so that
    the sharded optimizer state, gradient reduction, offload, checkpoints and the trainer -> rollout weight
    sync treat them like every other block.  The reference trains the tower with the rest of the HF model
    under FSDP (chatlearn/models/fsdp_module.py:250-295).  Leaves carry the HF names (``visual.*``); the
    patch-embedding kernel stays flattened to a matrix."""
    from .layout import _full
    from .model import ParamBlock
    if "vision" in lm.block_by_name:
        return lm.block_by_name["vision"]
    leaves = [_full(k, tuple(p.shape), k) for k, p in tower.params.items()]
    blk = ParamBlock("vision", leaves, tower.dtype, tower.device, pad_to)
    with torch.no_grad():
        for k, p in tower.params.items():
            blk.params[k].copy_(p)
    tower.params = blk.params                  # the same dict: re-bound leaves (offload, autograd) stay visible
    tower.trainable = True
    lm.blocks.append(blk)
    lm.block_by_name["vision"] = blk
    # HF keeps the patch embedding as a convolution kernel [hidden, channels, frames, patch, patch]
    a = tower.arch
    lm.hf_reshape = {"visual.patch_embed.proj.weight": (a.hidden_size, a.in_channels, a.temporal_patch_size,
                                                        a.patch_size, a.patch_size)}
    return blk


def multimodal_inputs(lm, tower, tokens: torch.Tensor, seq_lens, mm, ctx, with_embeddings: bool = True):
    """Input embeddings and (time, row, column) positions of a packed row whose samples may carry
    images or videos.  ``mm[i] = (pixel_values, image_grid_thw[, visual_time_steps])`` or ``(None, None)`` per
    sample (grids of all images and videos in the order of their placeholder runs); segments
    past ``len(mm)`` (alignment padding) count up from zero.  Sets ``ctx.mrope_positions`` and
    returns the embeddings (image placeholder rows replaced by the tower's output)."""
    from .model import embed
    arch = lm.arch
    itok, vtok, merge = arch.image_token_id, arch.video_token_id, tower.arch.spatial_merge_size
    host = tokens.detach().cpu()
    pos, px, grids, rows, off = [], [], [], [], 0
    for i, L in enumerate(seq_lens):
        seg = host[off:off + L]
        pv, g, steps = (tuple(mm[i]) + (None,))[:3] if i < len(mm) else (None, None, None)
        if pv is not None and len(g):
            g = g.tolist() if torch.is_tensor(g) else [list(v) for v in g]
            p3, _ = mrope_positions(seg, g, itok, merge, vtok, steps)
            px.append(torch.as_tensor(pv))
            grids.extend(g)
            # the rows of this sample's images: its first placeholder tokens, as many as it has merged patches
            # (a placeholder token the model generated later in the response is an ordinary token)
            vis = (seg == itok) | (seg == vtok) if vtok is not None else seg == itok
            want = sum(int(t) * int(h) * int(w) for t, h, w in g) // (merge * merge)
            mine = vis.nonzero(as_tuple=True)[0][:want]
            assert mine.numel() == want, f"{mine.numel()} image / video tokens but {want} embeddings in sample {i}"
            rows.append(mine + off)
        else:
            p3 = torch.arange(L).view(1, -1).expand(3, -1)
        pos.append(p3)
        off += L
    ctx.mrope_positions = torch.cat(pos, 1).contiguous().to(tokens.device)
    if not with_embeddings:            # later pipeline stages need the positions only
        return None
    x = embed(lm.block_by_name["embed"].params, tokens, ctx).to(lm.dtype)
    if px:
        # a tower whose weights are a parameter block of the model (attach_vision_block) is trained with it
        with torch.set_grad_enabled(torch.is_grad_enabled() and getattr(tower, "trainable", False)):
            img = tower(torch.cat(px, 0).to(tokens.device), grids)
        taps = []
        if isinstance(img, tuple):
            img, taps = img
        img = img.to(x.dtype)
        rows = torch.cat(rows).to(tokens.device)
        assert rows.numel() == img.shape[0], f"{rows.numel()} image / video tokens but {img.shape[0]} embeddings"
        x = x.index_put((rows,), img)                  # out of place: the embedding rows stay differentiable
        if taps:
            ctx.deepstack = (rows, [t.to(x.dtype) for t in taps])
    return x
