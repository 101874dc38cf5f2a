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
  generated so far), so nothing is ever lost and no swap space is needed;
* prefix sharing: the full KV blocks of a prompt are published under a hash of the
  tokens they cover (chained over the blocks before them).  A later request whose
  prompt starts with the same tokens adopts those blocks by reference instead of
  computing them: GRPO samples every prompt ``num_inference_per_prompt`` times, so
  all but one sample of a group skip the prompt's prefill, the group's prompt KV
  exists once, and the decode kernels of the group read the same physical blocks
  (which the L2 then serves).  Shared blocks are never written again: only whole
  blocks are shared and at least one prompt token is always left for the adopter
  to compute, so no copy-on-write is needed.  An adopter waits while the blocks
  it could share are still being computed by the request that owns them.
"""
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional


class BlockAllocator:
    """Free list with reference counts: a block shared by several sequences returns to the pool when the
    last of them lets go (``on_release`` is then told, so the prefix table can forget it)."""

    def __init__(self, num_blocks: int, block_size: int):
        self.num_blocks, self.block_size = num_blocks, block_size
        self._free: List[int] = list(range(num_blocks - 1, -1, -1))
        self._ref: List[int] = [0] * num_blocks
        self.on_release = None

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        assert n <= len(self._free), "out of KV blocks"
        out = [self._free.pop() for _ in range(n)]
        for b in out:
            self._ref[b] = 1
        return out

    def share(self, blocks: List[int]):
        for b in blocks:
            assert self._ref[b] > 0, "sharing a block nobody holds"
            self._ref[b] += 1

    def free(self, blocks: List[int]):
        for b in reversed(blocks):
            self._ref[b] -= 1
            if self._ref[b] == 0:
                self._free.append(b)
                if self.on_release is not None:
                    self.on_release(b)

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
    # tokens sampled on the device whose values the host has not read yet (pipelined decode: 0 or 1); they
    # count for block allocation and positions, their values arrive one step later
    inflight: int = 0

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
                 max_num_batched_tokens: int = 32768, prefix_sharing: bool = True):
        self.alloc = BlockAllocator(num_blocks, block_size)
        self.max_num_seqs = max_num_seqs
        self.max_tokens = max_num_batched_tokens
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.stats = {"preemptions": 0, "steps": 0, "prefill_tokens": 0, "decode_tokens": 0,
                      "shared_prefix_tokens": 0}
        # prefix table: chained hash of a full block's tokens -> {"block", "tokens", "owner"}; ``owner`` is the
        # sequence still computing the block (None once its KV is complete)
        self.prefix_sharing = prefix_sharing
        self._prefix: Dict[int, dict] = {}
        self._block_key: Dict[int, int] = {}
        self.alloc.on_release = self._forget_block

    def add(self, seq: Sequence):
        self.waiting.append(seq)

    # ------------------------------------------------------------------ prefix sharing
    def _forget_block(self, block: int):
        key = self._block_key.pop(block, None)
        if key is not None:
            self._prefix.pop(key, None)

    def _keys(self, s: Sequence):
        """(key, tokens) of every full block of the sequence's current tokens, chained over the blocks before."""
        toks = s.tokens
        cached = getattr(s, "_pkeys", None)
        if cached is not None and cached[0] == len(toks):
            return cached[1]
        bs, out, prev = self.alloc.block_size, [], 0
        for i in range(len(toks) // bs):
            t = tuple(toks[i * bs:(i + 1) * bs])
            prev = hash((prev, t))
            out.append((prev, t))
        s._pkeys = (len(toks), out)
        return out

    def _publish(self, s: Sequence):
        """Offer the full blocks this sequence holds (and is computing, or has computed) to later requests."""
        if not self.prefix_sharing or s.mm is not None:
            return
        keys = self._keys(s)
        for i in range(min(len(keys), len(s.blocks))):
            k, t = keys[i]
            if k not in self._prefix and s.blocks[i] not in self._block_key:
                self._prefix[k] = {"block": s.blocks[i], "tokens": t, "owner": s}
                self._block_key[s.blocks[i]] = k

    def _settle(self, s: Sequence):
        """The sequence stops computing (finished or preempted): what it completed stays on offer for as long as
        somebody holds the block, what it left unfinished is withdrawn."""
        bs = self.alloc.block_size
        for i, b in enumerate(s.blocks):
            k = self._block_key.get(b)
            e = self._prefix.get(k) if k is not None else None
            if e is not None and e["owner"] is s:
                if s.num_computed >= (i + 1) * bs:
                    e["owner"] = None
                else:
                    del self._prefix[k]
                    del self._block_key[b]

    def _shareable(self, s: Sequence):
        """``(n, pending)``: how many leading full blocks of the request are on offer and complete, and whether
        the next one is still being computed by its owner."""
        if not self.prefix_sharing or not self._prefix or s.num_computed != 0 or s.blocks or s.mm is not None:
            return 0, False
        bs = self.alloc.block_size
        keys = self._keys(s)
        limit = (s.length - 1) // bs                   # leave at least one token to compute: its logits are needed
        n = 0
        for i in range(min(limit, len(keys))):
            k, t = keys[i]
            e = self._prefix.get(k)
            if e is None or e["tokens"] != t:
                break
            if e["owner"] is not None:
                if e["owner"].num_computed >= (i + 1) * bs:
                    e["owner"] = None
                else:
                    return n, True
            n += 1
        return n, False

    def _adopt_prefixes(self):
        """Waiting requests whose prompt starts with published blocks take them by reference and enter the
        running set with those tokens counted as computed; a request whose prefix is still being computed by
        its owner keeps waiting (it must not start computing the same blocks itself)."""
        if not self.prefix_sharing or not self._prefix:
            return
        bs = self.alloc.block_size
        for s in list(self.waiting):
            n, pending = self._shareable(s)
            if pending or n == 0 or len(self.running) >= self.max_num_seqs:
                continue
            keys = self._keys(s)
            blocks = [self._prefix[keys[i][0]]["block"] for i in range(n)]
            self.alloc.share(blocks)
            s.blocks = blocks
            s.num_computed = n * bs
            self.waiting.remove(s)
            self.running.append(s)
            self.stats["shared_prefix_tokens"] += n * bs

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
            self._settle(victim)
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
        self._adopt_prefixes()
        # --- admission / chunked prefill ---
        budget = self.max_tokens
        seqs, q_lens, samples = [], [], []
        # sequences already admitted but with prompt KV still missing come first
        partial = [s for s in self.running if s.length + s.inflight - s.num_computed > 1]
        for s in partial:
            if budget <= 0:
                break
            todo = s.length - s.num_computed
            n = min(todo, budget)
            if not self._ensure_blocks(s, s.num_computed + n):
                break
            self._publish(s)
            seqs.append(s); q_lens.append(n); samples.append(n == todo)
            budget -= n
        # A step is either all "fresh" (every sequence starts at position 0: packed attention over the
        # step's own keys) or all continuation chunks (attention over the paged cache): new prompts are
        # not admitted next to a continuation, and a prompt is only cut when it can never fit whole.
        fresh_ok = not seqs
        at = 0
        while fresh_ok and at < len(self.waiting) and budget > 0 and len(self.running) < self.max_num_seqs:
            s = self.waiting[at]
            n_ready, pending = self._shareable(s)
            if pending or n_ready > 0:
                # its prefix is being computed by another request (possibly one admitted a moment ago in this
                # very step), or is ready to be adopted at the next step: it does not start from position 0
                at += 1
                continue
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
            del self.waiting[at]
            self.running.append(s)
            self._publish(s)
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
            while not self._ensure_blocks(s, s.length + s.inflight):
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
        self._settle(seq)
        self.alloc.free(seq.blocks)
        seq.blocks = []
