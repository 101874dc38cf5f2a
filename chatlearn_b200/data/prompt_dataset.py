"""Prompt datasets: raw records → the per-sample dict the rollout consumes.

Parity: chatlearn/data/prompt_dataset.py:34-95 (``PromptPipeline``) and the VLM
variant chatlearn/data/vl_prompt_dataset.py.  Sample schema produced here:
``{input_ids, prompt, prompt_token_length, prompt_token_ids, data_source,
ground_truth, agent_name, agent_cfg_path}`` (or ``messages`` when ``raw_chat``).
A record may already carry ``input_ids`` (synthetic token-id prompts); those are
used as they are and need no tokenizer.
"""
from typing import Any, Dict, List, Optional


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
    """Vision-language prompts: same schema plus ``pixel_values``,
    ``image_grid_thw`` and ``multi_modal_data`` passed through from the record
    (pre-extracted features; no image decoding is done here)."""

    def __init__(self, data_list, max_prompt_tokens_length, tokenizer=None, processor=None,
                 enable_thinking=False, raw_chat=False):
        super().__init__(data_list, max_prompt_tokens_length, tokenizer, enable_thinking, raw_chat)
        kept = {id(s): s for s in self.data}
        j = 0
        for item in data_list:
            if j >= len(self.data):
                break
            s = self.data[j]
            for k in ("pixel_values", "image_grid_thw", "multi_modal_data", "images"):
                if k in item:
                    s[k] = item[k]
            j += 1
        del kept
