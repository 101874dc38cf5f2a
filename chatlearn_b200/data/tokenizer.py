"""Tokenizers usable without network access.

``NullTokenizer`` maps text of space-separated integers to ids and back (the
role Megatron's ``NullTokenizer`` plays in chatlearn/configs/megatron_config.py
``tokenizer_type``); ``ByteTokenizer`` is a reversible UTF-8 byte tokenizer for
rule rewards on real text.  ``load_tokenizer`` returns a HuggingFace tokenizer
when a tokenizer directory exists, else falls back to these.
"""
import os
from typing import List, Optional


class NullTokenizer:
    def __init__(self, vocab_size: int = 32000, eos_token_id: Optional[int] = None):
        self.vocab_size = vocab_size
        self.eos_token_id = vocab_size - 1 if eos_token_id is None else eos_token_id
        self.pad_token_id = self.eos_token_id
        self.eos_token = str(self.eos_token_id)

    def encode(self, text: str, **_) -> List[int]:
        return [int(t) % self.vocab_size for t in text.split()]

    def decode(self, ids, skip_special_tokens: bool = False, **_) -> str:
        ids = ids.tolist() if hasattr(ids, "tolist") else list(ids)
        if skip_special_tokens:
            ids = [i for i in ids if i != self.eos_token_id]
        return " ".join(str(int(i)) for i in ids)

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True, **_):
        text = " ".join(m["content"] if isinstance(m, dict) else str(m) for m in messages)
        return self.encode(text) if tokenize else text

    def __len__(self):
        return self.vocab_size


class ByteTokenizer:
    """ids 0..255 are bytes, 256 = BOS, 257 = EOS; vocab may be padded above that."""

    def __init__(self, vocab_size: int = 512):
        assert vocab_size >= 258
        self.vocab_size = vocab_size
        self.bos_token_id, self.eos_token_id = 256, 257
        self.pad_token_id = self.eos_token_id
        self.eos_token = "<eos>"

    def encode(self, text: str, **_) -> List[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids, skip_special_tokens: bool = True, **_) -> str:
        ids = ids.tolist() if hasattr(ids, "tolist") else list(ids)
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True, **_):
        parts = []
        for m in messages:
            parts.append(f"<|{m.get('role', 'user')}|>\n{m.get('content', '')}\n")
        if add_generation_prompt:
            parts.append("<|assistant|>\n")
        text = "".join(parts)
        return self.encode(text) if tokenize else text

    def __len__(self):
        return self.vocab_size


def load_tokenizer(path: Optional[str], vocab_size: int = 32000, kind: str = "auto"):
    if kind == "null":
        return NullTokenizer(vocab_size)
    if kind == "byte":
        return ByteTokenizer(max(vocab_size, 258))
    if path and os.path.isdir(path) and any(
            os.path.exists(os.path.join(path, f)) for f in ("tokenizer.json", "tokenizer.model", "vocab.json")):
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(path, trust_remote_code=True)
    return NullTokenizer(vocab_size)
