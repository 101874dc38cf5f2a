"""Extraction of tool calls from generated text.

Parity: chatlearn/models/agent/tool_parser.py:24-112 (parser registry and the
Hermes ``<tool_call>{json}</tool_call>`` format).  Synchronous: parsing runs between
two batched generation turns, so there is no event loop to yield to.
"""
import json
import re
from dataclasses import dataclass
from typing import Dict, List, Tuple, Type

from chatlearn_b200.utils.logger import logger


@dataclass
class FunctionCall:
    name: str
    arguments: str          # JSON text as generated (may be invalid; validate before use)


class ToolParser:
    _registry: Dict[str, Type["ToolParser"]] = {}

    def __init__(self, tokenizer):
        self.tokenizer = tokenizer

    def extract_tool_calls(self, response_ids: List[int]) -> Tuple[str, List[FunctionCall]]:
        """Returns (text without the tool-call blocks, calls in order of appearance)."""
        raise NotImplementedError

    @classmethod
    def register(cls, name: str):
        def deco(sub):
            cls._registry[name] = sub
            return sub
        return deco

    @classmethod
    def get_tool_parser(cls, name: str, tokenizer) -> "ToolParser":
        if name not in cls._registry:
            raise ValueError(f"unknown tool parser {name!r}; known: {sorted(cls._registry)}")
        return cls._registry[name](tokenizer)


@ToolParser.register("hermes")
class HermesToolParser(ToolParser):
    OPEN, CLOSE = "<tool_call>", "</tool_call>"
    _block = re.compile(r"<tool_call>(.*?)</tool_call>", re.DOTALL)

    def extract_tool_calls(self, response_ids):
        text = self.tokenizer.decode(response_ids)
        return self.extract_from_text(text)

    def extract_from_text(self, text: str):
        if self.OPEN not in text or self.CLOSE not in text:
            return text, []
        calls = []
        for body in self._block.findall(text):
            try:
                obj = json.loads(body)
                calls.append(FunctionCall(obj["name"], json.dumps(obj["arguments"], ensure_ascii=False)))
            except Exception as e:  # malformed JSON or missing keys: the call is dropped
                logger.warning(f"tool call could not be decoded: {e}")
        return self._block.sub("", text), calls
