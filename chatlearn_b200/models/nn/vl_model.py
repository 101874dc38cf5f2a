"""Vision-language causal LM: vision tower + language model with multimodal rotary positions.

Parity: the Qwen2.5-VL path the reference trains through HuggingFace
(chatlearn/models/patches/transformers/qwen2_5_vl_patch.py; data contract of
chatlearn/data/vl_prompt_dataset.py: ``pixel_values`` + ``image_grid_thw`` per sample).  The
language model is this package's ``CausalLM`` (flat parameter blocks, so ZeRO sharding, checkpoints
and weight sync apply to it unchanged); the tower's weights are kept by HF name.  Image embeddings
replace the embeddings of the image placeholder tokens; positions are (time, row, column) triples.
"""
from typing import Dict, Sequence

import torch

from .arch import ModelArch
from .model import CausalLM, FwdCtx
from .vision import build_vision_tower, mrope_positions


def strip_language_prefix(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """HF vision-language checkpoints name the language model ``model.language_model.*``."""
    out = {}
    for k, v in sd.items():
        if k.startswith("model.language_model."):
            out["model." + k[len("model.language_model."):]] = v
        elif not k.startswith("model.visual.") and not k.startswith("visual."):
            out[k] = v
    return out


class VLCausalLM:
    def __init__(self, arch: ModelArch, dtype=torch.float32, device="cpu", **lm_kwargs):
        assert arch.vision_config is not None and arch.mrope_section is not None and arch.image_token_id is not None, \
            "a vision-language architecture needs vision_config, mrope_section and image_token_id"
        self.arch = arch
        self.lm = CausalLM(arch, dtype=dtype, device=device, **lm_kwargs)
        self.visual = build_vision_tower(arch, dtype, device)
        self.varch = self.visual.arch

    def init_weights(self, seed: int = 0):
        self.lm.init_weights(seed)
        self.visual.init_weights(seed + 1)
        return self

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor]):
        self.lm.load_hf_state_dict(strip_language_prefix(sd))
        self.visual.load_hf_state_dict(sd)

    def positions(self, input_ids: torch.Tensor, image_grid_thw, time_steps=None) -> torch.Tensor:
        pos, _ = mrope_positions(input_ids.cpu(), image_grid_thw, self.arch.image_token_id, self.varch.spatial_merge_size,
                                 self.arch.video_token_id, time_steps)
        return pos.to(input_ids.device)

    def hidden_states(self, tokens, ctx: FwdCtx, pixel_values=None, image_grid_thw=None, layer_hook=None):
        """``tokens`` is a packed row; ``ctx.mrope_positions`` must hold the [3, T] positions (see
        ``packed_positions``).  Image placeholder rows take the tower's embeddings (and, for towers with
        deep-stack taps, the early layers add the tap features at those rows)."""
        from .model import embed
        x = embed(self.lm.block_by_name["embed"].params, tokens, ctx).to(self.lm.dtype)
        if pixel_values is not None and pixel_values.numel():
            img = self.visual(pixel_values.to(x.device), image_grid_thw)
            taps = []
            if isinstance(img, tuple):
                img, taps = img
            vis = tokens == self.arch.image_token_id
            if self.arch.video_token_id is not None:
                vis = vis | (tokens == self.arch.video_token_id)
            rows = vis.nonzero(as_tuple=True)[0][:img.shape[0]]     # (placeholder ids generated later on are text)
            assert rows.numel() == img.shape[0], f"{rows.numel()} image / video placeholder tokens but {img.shape[0]} embeddings"
            x = x.index_put((rows,), img.to(x.dtype))
            if taps:
                ctx.deepstack = (rows, taps)
        return self.lm.hidden_states(tokens, ctx, layer_hook, x=x)

    def packed_positions(self, seqs: Sequence[torch.Tensor], grids: Sequence) -> torch.Tensor:
        """[3, T] positions of sequences packed back to back (each restarts at zero)."""
        parts = [self.positions(s, g) for s, g in zip(seqs, grids)]
        return torch.cat(parts, 1)

    def logits(self, tokens, ctx, pixel_values=None, image_grid_thw=None):
        return self.lm.logits(self.hidden_states(tokens, ctx, pixel_values, image_grid_thw))

    def logprobs(self, tokens, labels, ctx, pixel_values=None, image_grid_thw=None, temperature=1.0):
        from chatlearn_b200 import ops
        h = self.hidden_states(tokens, ctx, pixel_values, image_grid_thw)
        return ops.lmhead_logprob_entropy(h, self.lm.lm_head_weight(), labels, temperature)
