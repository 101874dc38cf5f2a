"""Prompt datasets: raw records → the per-sample dict the rollout consumes.

Parity: chatlearn/data/prompt_dataset.py:34-95 (``PromptPipeline``) and the VLM
variant chatlearn/data/vl_prompt_dataset.py.  Sample schema produced here:
``{input_ids, prompt, prompt_token_length, prompt_token_ids, data_source,
ground_truth, agent_name, agent_cfg_path}`` (or ``messages`` when ``raw_chat``).
A record may already carry ``input_ids`` (synthetic token-id prompts); those are
used as they are and need no tokenizer.
"""
from typing import Any, Dict, List


class PromptPipeline:
    def __init__(self, data_list: List[Dict[str, Any]], max_prompt_tokens_length: int,
                 tokenizer=None, enable_thinking: bool = False, raw_chat: bool = False):
        self.tokenizer = tokenizer
        self.data: List[Dict[str, Any]] = []
        self.max_prompt = 0
        for item in data_list:
            rm = item.get("reward_model") or {}
            sample = {
                "data_source": item.get("data_source", ""),
                "ground_truth": rm.get("ground_truth", item.get("ground_truth")),
                "agent_name": item.get("agent_name"),
                "agent_cfg_path": item.get("agent_cfg_path"),
            }
            prompt = item.get("prompt")
            if raw_chat:
                sample["messages"] = prompt
                self.data.append(sample)
                continue
            if item.get("input_ids") is not None:
                ids = [int(t) for t in item["input_ids"]]
                if prompt is None:
                    prompt = " ".join(map(str, ids))
            else:
                assert tokenizer is not None, "text prompts need a tokenizer"
                if isinstance(prompt, list):
                    prompt = tokenizer.apply_chat_template(
                        prompt, tokenize=False, add_generation_prompt=True,
                        enable_thinking=enable_thinking)
                ids = list(tokenizer.encode(prompt))
            sample.update(input_ids=ids, prompt=prompt, prompt_token_length=len(ids),
                          prompt_token_ids=ids)
            self.max_prompt = max(self.max_prompt, len(ids))
            if len(ids) < max_prompt_tokens_length:   # strict, as in the reference
                self.data.append(sample)
        self.valid_ratio = len(self.data) / max(len(data_list), 1)

    def __getitem__(self, ix: int):
        return self.data[ix]

    def __len__(self) -> int:
        return len(self.data)

    def collate_fn(self, samples):
        return samples


class VLPromptPipeline(PromptPipeline):
    """Vision-language prompts (chatlearn/data/vl_prompt_dataset.py).  A record carries either
    pre-extracted ``pixel_values`` + ``image_grid_thw``, or ``images`` (paths, bytes or PIL images),
    which are resized, normalised and cut into patches here (``data/vision_utils.py``).  Every image
    placeholder token of the prompt is expanded to one token per merged patch of its image, so the
    rollout engine and the trainers can drop the vision tower's embeddings into place.  ``videos`` (per video a
    list of frames, ``{"frames": [...], "fps": f}``, a file path or ``{"path": ..., "fps": rate}``) go the same way behind their own placeholder token: images
    and videos share ``pixel_values`` / ``image_grid_thw`` in the order of their placeholders, and
    ``visual_time_steps`` holds per item the temporal position step (``None`` for images).  Sample schema:
    the text schema plus ``pixel_values [patches, C·Tp·P·P]``, ``image_grid_thw [[t, h, w], ...]``."""

    def __init__(self, data_list, max_prompt_tokens_length, tokenizer=None, processor=None,
                 enable_thinking=False, raw_chat=False, image_token_id=None, merge_size: int = 2,
                 min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280, patch_size: int = 14,
                 temporal_patch_size: int = 2, mean=None, std=None, video_token_id=None,
                 tokens_per_second: float = 1.0, video_max_pixels: int = 14 * 14 * 4 * 320):
        # the length filter runs after the placeholder expansion, so filter here, not in the base class
        super().__init__(data_list, 1 << 30, tokenizer, enable_thinking, raw_chat)
        from chatlearn_b200.data.vision_utils import expand_image_tokens, process_images, process_visuals
        if image_token_id is None and tokenizer is not None and hasattr(tokenizer, "convert_tokens_to_ids"):
            image_token_id = tokenizer.convert_tokens_to_ids("<|image_pad|>")
        if video_token_id is None and tokenizer is not None and hasattr(tokenizer, "convert_tokens_to_ids"):
            video_token_id = tokenizer.convert_tokens_to_ids("<|video_pad|>")
        kept = []
        for item, s in zip(data_list, self.data):
            for k in ("pixel_values", "image_grid_thw", "multi_modal_data", "visual_time_steps"):
                if k in item:
                    s[k] = item[k]
            kw = dict(merge_size=merge_size, min_pixels=min_pixels, max_pixels=max_pixels, patch_size=patch_size,
                      temporal_patch_size=temporal_patch_size)
            if mean is not None:
                kw.update(mean=mean, std=std)
            if item.get("videos") and s.get("pixel_values") is None:
                # images and videos in the order of their placeholders in the tokenised prompt
                if "input_ids" in s:
                    assert image_token_id is not None and video_token_id is not None, \
                        "tokenised records with videos need the two placeholder token ids"
                    order, itok, vtok = s["input_ids"], image_token_id, video_token_id
                else:
                    # raw chat records are tokenised turn by turn later: their images come first, then their videos
                    itok, vtok = 0, 1
                    order = [itok] * len(item.get("images") or []) + [vtok] * len(item["videos"])
                pv, grids, steps = process_visuals(order, item.get("images"), item["videos"], itok, vtok,
                                                   tokens_per_second, video_kw=dict(max_pixels=video_max_pixels), **kw)
                s["pixel_values"], s["image_grid_thw"], s["visual_time_steps"] = pv, grids, steps
            elif item.get("images") and s.get("pixel_values") is None:
                pv, grid = process_images(item["images"], **kw)
                s["pixel_values"], s["image_grid_thw"] = pv, grid.tolist()
            if s.get("pixel_values") is not None and "input_ids" in s and image_token_id is not None:
                import torch
                s["pixel_values"] = torch.as_tensor(s["pixel_values"], dtype=torch.float32)
                grids = [list(map(int, g)) for g in s["image_grid_thw"]]
                n_merged = sum(t * h * w for t, h, w in grids) // (merge_size ** 2)
                n_place = s["input_ids"].count(image_token_id) + \
                    (s["input_ids"].count(video_token_id) if video_token_id is not None else 0)
                if n_place != n_merged:                                     # one placeholder per image / video so far
                    s["input_ids"] = expand_image_tokens(s["input_ids"], grids, image_token_id, merge_size, video_token_id)
                s["prompt_token_ids"] = s["input_ids"]
                s["prompt_token_length"] = len(s["input_ids"])
            if raw_chat or len(s.get("input_ids", [])) < max_prompt_tokens_length:
                kept.append(s)
        self.data = kept
        self.valid_ratio = len(kept) / max(len(data_list), 1)
