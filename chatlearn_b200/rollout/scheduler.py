"""Continuous-batching scheduler and paged KV block allocator.

This replaces the scheduling half of vLLM/SGLang that the reference drives
through ``llm.generate`` (chatlearn/models/vllm_module.py:360-411) and
``engine.async_generate`` (chatlearn/models/sglang_module.py:403-413).  Policy:

* waiting requests are admitted FCFS while KV blocks and the per-step token
  budget (``max_num_batched_tokens``) allow; long prompts are prefilled in
  chunks;
* every running sequence decodes one token per step;
* when the pool runs dry the youngest running sequence is preempted: its blocks
  are freed and it re-enters the waiting queue to be recomputed (prompt +
  generated so far), so nothing is ever lost and no swap space is needed.

A C++ implementation with the same interface (``native_sched``) is used when
the extension is built; this Python class is the specification and the CPU path.
"""
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple


class BlockAllocator:
    def __init__(self, num_blocks: int, block_size: int):
        self.num_blocks, self.block_size = num_blocks, block_size
        self._free: List[int] = list(range(num_blocks - 1, -1, -1))

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        assert n <= len(self._free), "out of KV blocks"
        out = [self._free.pop() for _ in range(n)]
        return out

    def free(self, blocks: List[int]):
        self._free.extend(reversed(blocks))

    def blocks_for(self, num_tokens: int) -> int:
        return (num_tokens + self.block_size - 1) // self.block_size


@dataclass
class Sequence:
    req_id: int
    prompt: List[int]
    max_new_tokens: int
    sampling: "object" = None
    output: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)
    blocks: List[int] = field(default_factory=list)
    num_computed: int = 0          # tokens whose KV is in the cache
    finished: bool = False
    finish_reason: Optional[str] = None
    preemptions: int = 0
    # vision-language requests: image embeddings and (time, row, column) positions of the prompt;
    # text after the images sits at position index + rope_delta
    mm: Optional[dict] = None
    rope_delta: int = 0

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def length(self) -> int:
        return len(self.prompt) + len(self.output)


@dataclass
class StepPlan:
    seqs: List[Sequence]
    q_lens: List[int]              # new tokens fed per sequence this step
    is_prefill: bool               # every sequence starts at position 0 this step
    samples: List[bool]            # whether a token is sampled for the sequence


class Scheduler:
    def __init__(self, num_blocks: int, block_size: int, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 32768):
        self.alloc = BlockAllocator(num_blocks, block_size)
        self.max_num_seqs = max_num_seqs
        self.max_tokens = max_num_batched_tokens
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.stats = {"preemptions": 0, "steps": 0, "prefill_tokens": 0, "decode_tokens": 0}

    def add(self, seq: Sequence):
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _ensure_blocks(self, seq: Sequence, upto_tokens: int) -> bool:
        need = self.alloc.blocks_for(upto_tokens) - len(seq.blocks)
        if need <= 0:
            return True
        if need > self.alloc.num_free:
            return False
        seq.blocks.extend(self.alloc.alloc(need))
        return True

    def _preempt_one(self, keep: Sequence) -> Optional[Sequence]:
        """Evict the youngest running sequence other than ``keep``; returns it."""
        for i in range(len(self.running) - 1, -1, -1):
            victim = self.running[i]
            if victim is keep:
                continue
            del self.running[i]
            self.alloc.free(victim.blocks)
            victim.blocks = []
            victim.num_computed = 0
            victim.preemptions += 1
            self.stats["preemptions"] += 1
            self.waiting.appendleft(victim)
            return victim
        return None

    def schedule(self) -> Optional[StepPlan]:
        """Next step: prefill work first (admission), else one decode step."""
        self.stats["steps"] += 1
        # --- admission / chunked prefill ---
        budget = self.max_tokens
        seqs, q_lens, samples = [], [], []
        # sequences already admitted but with prompt KV still missing come first
        partial = [s for s in self.running if s.length - s.num_computed > 1]
        for s in partial:
            if budget <= 0:
                break
            todo = s.length - s.num_computed
            n = min(todo, budget)
            if not self._ensure_blocks(s, s.num_computed + n):
                break
            seqs.append(s); q_lens.append(n); samples.append(n == todo)
            budget -= n
        # A step is either all "fresh" (every sequence starts at position 0: packed attention over the
        # step's own keys) or all continuation chunks (attention over the paged cache): new prompts are
        # not admitted next to a continuation, and a prompt is only cut when it can never fit whole.
        fresh_ok = not seqs
        while fresh_ok and self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            s = self.waiting[0]
            todo = s.length - s.num_computed
            if todo > budget and seqs:
                break
            n = min(todo, budget)
            # keep one block of head-room per running sequence so decode can proceed
            if self.alloc.blocks_for(s.num_computed + n) - len(s.blocks) > \
                    self.alloc.num_free - len(self.running):
                break
            if not self._ensure_blocks(s, s.num_computed + n):
                break
            self.waiting.popleft()
            self.running.append(s)
            seqs.append(s); q_lens.append(n); samples.append(n == todo)
            budget -= n
        if seqs:
            self.stats["prefill_tokens"] += sum(q_lens)
            start0 = all(s.num_computed == 0 for s in seqs)
            return StepPlan(seqs, q_lens, start0, samples)
        # --- decode ---
        if not self.running:
            if self.waiting:
                raise RuntimeError("KV cache too small for a single waiting request")
            return None
        # common case first: every running sequence gets its block without preemption
        # (linear in the batch; the preemption path below re-validates membership)
        gone = set()
        ready = []
        for s in list(self.running):
            if id(s) in gone:
                continue
            while not self._ensure_blocks(s, s.length):
                victim = self._preempt_one(keep=s)
                if victim is None:
                    raise RuntimeError("KV cache too small for one sequence")
                gone.add(id(victim))
            ready.append(s)
        if gone:
            ready = [s for s in ready if id(s) not in gone]
        self.stats["decode_tokens"] += len(ready)
        return StepPlan(ready, [1] * len(ready), False, [True] * len(ready))

    def finish(self, seq: Sequence, reason: str):
        seq.finished, seq.finish_reason = True, reason
        if seq in self.running:
            self.running.remove(seq)
        self.alloc.free(seq.blocks)
        seq.blocks = []
