"""The rollout (generation) engine: paged KV cache, continuous batching, sampling.

Takes the place of vLLM / SGLang in the reference
(chatlearn/models/vllm_module.py:169-216,360-411, chatlearn/models/sglang_module.py:250-315):
the engine owns a TP/EP-sharded copy of the policy weights in rollout layout, a
paged KV cache, a continuous-batching scheduler and the sampler.  Memory is
managed by tag like the reference's sleep/wake-up
(vllm_module.py:442-469): ``weights`` and ``kv_cache`` can be released and
re-created independently, so the trainer can use the memory between rollouts.
"""
import math
import os
import time
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence as Seq

import torch

from chatlearn_b200 import ops
from chatlearn_b200.models.nn.model import CausalLM, FwdCtx, KVCtx
from chatlearn_b200.utils import xfer
from chatlearn_b200.utils.constant import TAG_KV_CACHE, TAG_WEIGHTS
from .scheduler import Scheduler, Sequence, StepPlan


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int = 16
    stop_token_ids: Seq[int] = ()
    ignore_eos: bool = False

    @property
    def has_penalty(self):
        return (self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
                or self.repetition_penalty != 1.0)

    def key(self):
        return (self.temperature, self.top_p, self.top_k, self.min_p, self.presence_penalty,
                self.frequency_penalty, self.repetition_penalty)


class RolloutEngine:
    def __init__(self, model: CausalLM, tp_group=None, ep_group=None, block_size: int = 64,
                 num_blocks: Optional[int] = None, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 32768, gpu_memory_utilization: float = 0.8,
                 max_model_len: int = 4096, seed: int = 0, kv_dtype=None,
                 lockstep_group=None, use_cuda_graphs: bool = True, vision=None):
        self.model, self.arch = model, model.arch
        self.device = model.device
        self.vision = vision                 # models.nn.vision.VisionTower for vision-language models
        self._embed_patch = None
        self.tp, self.ep = tp_group, ep_group
        # tensor-parallel reductions by this package's own peer-memory kernels (fused with
        # the residual add and the next RMSNorm) instead of NCCL; collective construction
        self.tp_symm = None
        if tp_group is not None and tp_group.size > 1 and self.device.type == "cuda" \
                and ops.get_mode() == "native" and os.environ.get("CLB200_SYMM_TP", "1") != "0":
            from chatlearn_b200.parallel import symm_collectives
            self.tp_symm = symm_collectives.get(tp_group)
            if self.tp_symm is not None:
                tp_group.fast["all_reduce"] = self.tp_symm.all_reduce
        # expert-parallel dispatch / combine through peer memory instead of NCCL all-to-all
        self.ep_symm = None
        epg = getattr(ep_group, "group", None)
        if epg is not None and epg.size > 1 and self.device.type == "cuda" and ops.get_mode() == "native" \
                and self.arch.num_experts and self.arch.num_experts % epg.size == 0 \
                and os.environ.get("CLB200_SYMM_EP", "1") != "0":
            from chatlearn_b200.parallel import symm_mem
            if symm_mem.available() and epg.size <= 8:
                from chatlearn_b200.parallel.symm_moe import SymmMoE
                self.ep_symm = SymmMoE(epg, self.arch.num_experts, self.arch.hidden_size)
                pairs = int(max_num_batched_tokens) * int(self.arch.num_experts_per_tok)
                moe = self.ep_symm
                epg.fast["moe_dispatch_combine"] = \
                    lambda x, w13, w2, w, idx, E: moe.experts(x, w13, w2, w, idx, pairs_per_rank=pairs)
        self.block_size = block_size
        self.max_num_seqs = max_num_seqs
        self.max_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.util = gpu_memory_utilization
        self.kv_dtype = kv_dtype or model.dtype
        self._num_blocks_cfg = num_blocks
        self.k_cache: List[torch.Tensor] = []
        self.v_cache: List[torch.Tensor] = []
        self.lin_conv, self.lin_rec, self._state_slot, self._free_state_slots = [], [], {}, []
        self.num_blocks = 0
        self.gen = torch.Generator(device=self.device)
        self.gen.manual_seed(seed)
        self.stats: Dict[str, float] = {}
        self._req_counter = 0
        # ranks that exchange tokens inside a forward (expert parallel) must run the
        # same number of forwards: they agree on "anyone still busy" every step
        self.lockstep = lockstep_group
        # "emulate": the captured decode step's host side (persistent input buffers, cached block tables, input
        # tokens fed from the previous step's samples, read-back one step late) with the step's body run directly
        # instead of through a CUDA graph: the same logic on CPU ranks, where the tests exercise it
        self._emulate_graphs = use_cuda_graphs == "emulate"
        self.use_graphs = bool(use_cuda_graphs)
        self._graphs: Dict[Any, Any] = {}
        self._gs = None
        # pipelined decode: the step launched last whose sampled tokens the host has not read yet
        self._pending = None
        self._finished_buf: List[Sequence] = []
        self.pipelined = os.environ.get("CLB200_PIPELINED_DECODE", "1") != "0"

    # ------------------------------------------------------------------ memory
    def kv_bytes_per_block(self) -> int:
        a = self.arch
        tp = self.tp.size if self.tp is not None else 1
        if a.use_mla:
            per_tok = a.kv_lora_rank + a.qk_rope_head_dim       # one compressed row per token, shared by all heads
        else:
            from chatlearn_b200.models.nn.layout import kv_head_range
            nkv_l = kv_head_range(a, tp, 0)[1]
            per_tok = nkv_l * a.head_dim * 2
        esz = torch.empty((), dtype=self.kv_dtype).element_size()
        kv_layers = sum(1 for l in range(a.num_hidden_layers) if not a.layer_is_linear(l))
        return per_tok * esz * self.block_size * kv_layers

    def linear_state_bytes(self) -> int:
        """Convolution taps + recurrent matrix of every gated delta-net layer, for all state slots."""
        a = self.arch
        n_lin = sum(1 for l in range(a.num_hidden_layers) if a.layer_is_linear(l))
        if not n_lin:
            return 0
        kd, vd = a.linear_num_key_heads * a.linear_key_head_dim, a.linear_num_value_heads * a.linear_value_head_dim
        esz = torch.empty((), dtype=self.model.dtype).element_size()
        per_slot = (a.linear_conv_kernel_dim - 1) * (2 * kd + vd) * esz \
            + a.linear_num_value_heads * a.linear_key_head_dim * a.linear_value_head_dim * 4
        return n_lin * per_slot * (self.max_num_seqs + 2)

    def alloc_kv_cache(self):
        if self.k_cache:
            return
        a = self.arch
        tp = self.tp.size if self.tp is not None else 1
        nb = self._num_blocks_cfg
        if nb is None:
            if self.device.type == "cuda":
                free, total = torch.cuda.mem_get_info(self.device)
                budget = int(free - (1.0 - self.util) * total) - self.linear_state_bytes()
                nb = max(budget // self.kv_bytes_per_block(), 1)
            else:
                nb = 256
            # never more than what max_num_seqs full-length sequences can use
            cap = self.max_num_seqs * math.ceil(self.max_model_len / self.block_size) + 1
            nb = min(nb, cap)
            if self.tp is not None and self.tp.size > 1:
                t = torch.tensor([nb], device=self.device)
                import torch.distributed as dist
                dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.tp.pg)
                nb = int(t.item())
        self.num_blocks = nb
        if a.use_mla:
            nkv_l, dk, dv = 1, a.kv_lora_rank + a.qk_rope_head_dim, a.kv_lora_rank
        else:
            from chatlearn_b200.models.nn.layout import kv_head_range
            nkv_l = kv_head_range(a, tp, self.tp.rank if self.tp is not None else 0)[1]
            dk = dv = a.head_dim
        # one block beyond the allocator's range is scratch: padded rows of a captured
        # decode step write their (ignored) KV there
        self.lin_conv, self.lin_rec = [], []
        self._state_slot, self._free_state_slots = {}, list(range(self.max_num_seqs, -1, -1))
        for l in range(a.num_hidden_layers):
            if a.layer_is_linear(l):
                # gated delta-net layers keep a fixed-size state per sequence instead of keys and values
                # (of this tensor-parallel rank's heads)
                nk_l, nv_l = a.linear_num_key_heads // tp, a.linear_num_value_heads // tp
                kd, vd = nk_l * a.linear_key_head_dim, nv_l * a.linear_value_head_dim
                self.k_cache.append(torch.empty(0, device=self.device))
                self.v_cache.append(torch.empty(0, device=self.device))
                # slots 0..max_num_seqs are handed out; the last one is scratch for the padded rows of a captured step
                self.lin_conv.append(torch.zeros(self.max_num_seqs + 2, a.linear_conv_kernel_dim - 1, 2 * kd + vd,
                                                 dtype=self.model.dtype, device=self.device))
                self.lin_rec.append(torch.zeros(self.max_num_seqs + 2, nv_l, a.linear_key_head_dim,
                                                a.linear_value_head_dim, dtype=torch.float32, device=self.device))
                continue
            self.lin_conv.append(None)
            self.lin_rec.append(None)
            self.k_cache.append(torch.zeros(nb + 1, self.block_size, nkv_l, dk, dtype=self.kv_dtype,
                                            device=self.device))
            if a.use_mla:
                # the "values" of latent attention are the latent part of the same rows
                self.v_cache.append(self.k_cache[-1][..., :dv])
                continue
            self.v_cache.append(torch.zeros(nb + 1, self.block_size, nkv_l, dv, dtype=self.kv_dtype,
                                            device=self.device))
        self.invalidate_graphs()

    def free_kv_cache(self):
        self.invalidate_graphs()
        self.k_cache, self.v_cache = [], []
        self.lin_conv, self.lin_rec = [], []
        self.num_blocks = 0

    def _linear_state(self, seqs) -> Optional[Any]:
        """State slots of this step's sequences (assigned on first sight, reclaimed from finished or
        preempted sequences) and which of them start from an empty state."""
        if self.arch.layer_types is None:
            return None
        from chatlearn_b200.models.nn.hybrid import LinearState
        slots = self._state_slots_of(seqs)
        fresh = [s.num_computed == 0 for s in seqs]
        dev = self.device
        return LinearState(self.lin_conv, self.lin_rec,
                           xfer.to_device(torch.tensor(slots, dtype=torch.long), dev, "lin_slots"),
                           xfer.to_device(torch.tensor(fresh, dtype=torch.bool), dev, "lin_fresh"))

    def _state_slots_of(self, seqs) -> List[int]:
        live = {id(s) for s in seqs}
        slots = []
        for s in seqs:
            slot = self._state_slot.get(id(s))
            if slot is None:
                if not self._free_state_slots:
                    for key, (sl, other) in list(self._state_slot.items()):
                        if key not in live and (other.finished or other.num_computed == 0):
                            del self._state_slot[key]
                            self._free_state_slots.append(sl)
                assert self._free_state_slots, "more running sequences than state slots"
                slot = (self._free_state_slots.pop(), s)
                self._state_slot[id(s)] = slot
            slots.append(slot[0])
        return slots

    # ------------------------------------------------------------------ one step
    def _build_inputs(self, plan: StepPlan):
        bs = self.block_size
        toks, pos, slots, cu = [], [], [], [0]
        max_blocks = max(len(s.blocks) for s in plan.seqs)
        bt = torch.zeros(len(plan.seqs), max_blocks, dtype=torch.int32)
        seq_lens, last_rows = [], []
        # vision-language prompts: rows of an image prompt carry (time, row, column) positions and take
        # their embeddings from the vision tower; every later row sits at index + rope_delta
        any_mm = any(s.mm is not None and s.num_computed < len(s.prompt) for s in plan.seqs)
        pos3, patch_rows, patch_src = ([], [], []) if any_mm else (None, None, None)
        for i, (s, n) in enumerate(zip(plan.seqs, plan.q_lens)):
            start = s.num_computed
            all_t = s.tokens
            toks.extend(all_t[start:start + n])
            npr = len(s.prompt) if s.mm is not None else 0
            pos.extend(p if p < npr else p + s.rope_delta for p in range(start, start + n))
            if any_mm:
                row0 = cu[-1]
                if s.mm is not None and start < npr:
                    hi = min(start + n, npr)
                    pos3.append(s.mm["pos3"][:, start:hi])
                    for p in range(start, hi):
                        o = s.mm["ordinal"].get(p)
                        if o is not None:
                            patch_rows.append(row0 + p - start)
                            patch_src.append((s, o))
                    if hi < start + n:
                        tail = torch.arange(hi, start + n) + s.rope_delta
                        pos3.append(tail.view(1, -1).expand(3, -1))
                else:
                    tail = torch.arange(start, start + n) + s.rope_delta
                    pos3.append(tail.view(1, -1).expand(3, -1))
            for p in range(start, start + n):
                slots.append(s.blocks[p // bs] * bs + p % bs)
            bt[i, :len(s.blocks)] = torch.tensor(s.blocks, dtype=torch.int32)
            seq_lens.append(start + n)
            cu.append(cu[-1] + n)
            last_rows.append(cu[-1] - 1)
        dev = self.device
        # one pinned staging slot per input so the async copies never alias
        t = lambda x, dt, slot: xfer.to_device(torch.tensor(x, dtype=dt), dev, slot)  # noqa: E731
        kv = KVCtx(self.k_cache, self.v_cache, t(slots, torch.long, "slots"), xfer.to_device(bt, dev, "bt"),
                   t(seq_lens, torch.int32, "seq_lens"), t(plan.q_lens, torch.int32, "q_lens"), plan.is_prefill,
                   lin=self._linear_state(plan.seqs))
        ctx = FwdCtx(positions=t(pos, torch.long, "pos"), cu_seqlens=t(cu, torch.int32, "cu"),
                     max_seqlen=max(plan.q_lens), kv=kv, tp=self.tp, ep=self.ep, tp_symm=self._symm(), fuse_add_norm=True)
        self._embed_patch = None
        if any_mm:
            ctx.mrope_positions = xfer.to_device(torch.cat(pos3, 1).contiguous(), dev, "pos3")
            if patch_rows:
                src = torch.stack([s.mm["embeds"][o] for s, o in patch_src])
                rows_t = torch.tensor(patch_rows, dtype=torch.long, device=dev)
                self._embed_patch = (rows_t, src)
                levels = max(len(s.mm["deepstack"]) for s, _ in patch_src)
                if levels:
                    ctx.deepstack = (rows_t, [torch.stack([s.mm["deepstack"][lv][o] for s, o in patch_src])
                                              for lv in range(levels)])
        return t(toks, torch.long, "toks"), ctx, t(last_rows, torch.long, "last")

    def _symm(self):
        if self.tp_symm is not None:
            self.tp_symm.begin_forward()
        return self.tp_symm

    @torch.no_grad()
    def _logits(self, hidden_last):
        w = self.model.lm_head_weight()
        logits = None
        if hidden_last.is_cuda and ops.get_mode() == "native" and hidden_last.dtype == torch.bfloat16:
            # fp32 logits straight from the GEMM's accumulators: the trainer scores the same tokens from fp32 logits,
            # and a bf16 round trip here showed up as a rollout / trainer log-prob difference
            from chatlearn_b200.ops import native
            h2 = hidden_last.contiguous()
            if h2.shape[0] > 0 and native.get_gemm_impl() == "tcgen05" and native._gemm_ok(h2, w):
                logits = native.gemm_nt(h2, w, out_fp32=True)
        if logits is None:
            logits = ops.linear(hidden_last, w).float()
        if self.tp is not None and self.tp.size > 1 and w.shape[0] != self.arch.vocab_size:
            logits = self.tp.all_gather_cat(logits, dim=1)
        return logits

    # ------------------------------------------------------------------ CUDA-graph decode
    _BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 160, 192, 224, 256, 320, 384, 512)

    def _graph_state(self):
        """Persistent device inputs/outputs of the captured decode step."""
        if self._gs is None:
            dev, n = self.device, max(self.max_num_seqs, 1)
            n = min(b for b in self._BUCKETS if b >= n) if n <= self._BUCKETS[-1] else n
            width = math.ceil(self.max_model_len / self.block_size)
            z = lambda dt, *shape: torch.zeros(*shape, dtype=dt, device=dev)  # noqa: E731
            pin = dev.type == "cuda"
            # rows: token (when the host knows it), position, KV slot, sequence length, and for a token that is
            # still on the device its row in the previous step's batch plus a flag
            in64 = z(torch.long, 6, n)
            self._gs = dict(n=n, width=width, in64=in64, tokens=z(torch.long, n), pos=in64[1],
                            slots=in64[2], seq_lens=z(torch.int32, n), bt=z(torch.int32, n, width),
                            u=z(torch.float32, n), ids=z(torch.long, n), lp=z(torch.float32, n),
                            stage=torch.zeros(6, n, dtype=torch.int64, pin_memory=pin),
                            out_dev=[z(torch.float32, 2, n) for _ in range(2)],
                            out_host=[torch.zeros(2, n, dtype=torch.float32, pin_memory=pin) for _ in range(2)],
                            out_event=[torch.cuda.Event() for _ in range(2)] if dev.type == "cuda" else [None, None],
                            parity=0,
                            bt_host=torch.zeros(n, width, dtype=torch.int32, pin_memory=pin),
                            bt_len=[0] * n, bt_owner=[None] * n,
                            # sequences that share their first KV blocks (the samples of one prompt): up to n / 2
                            # groups of up to 8 rows each, the shared block count per group, and per row the first
                            # block that is its own
                            grp_q=torch.full((max(n // 2, 1), 8), -1, dtype=torch.int32, device=dev),
                            grp_nblk=z(torch.int32, max(n // 2, 1)), blk_start=z(torch.int32, n),
                            grp_stage=torch.zeros(max(n // 2, 1) * 9 + n, dtype=torch.int32, pin_memory=pin),
                            grp_key=None)
            if self.arch.layer_types is not None:
                # recurrent-state layers: the state slot of every row (decode rows never start fresh)
                self._gs.update(lin_slots=z(torch.long, n), lin_fresh=z(torch.bool, n),
                                lin_stage=torch.zeros(n, dtype=torch.int64, pin_memory=pin))
        return self._gs

    def invalidate_graphs(self):
        """Captured graphs hold raw pointers to the KV cache and the weights."""
        self._graphs = {}
        if self._gs is not None:
            self._gs["bt_owner"] = [None] * self._gs["n"]

    def _decode_body(self, B: int, sp):
        gs = self._gs
        kv = KVCtx(self.k_cache, self.v_cache, gs["slots"][:B], gs["bt"][:B], gs["seq_lens"][:B], None, False)
        if gs.get("use_groups"):
            kv.groups = (gs["grp_q"][:max(B // 2, 1)], gs["grp_nblk"][:max(B // 2, 1)], gs["blk_start"][:B])
        if self.arch.layer_types is not None:
            from chatlearn_b200.models.nn.hybrid import LinearState
            kv.lin = LinearState(self.lin_conv, self.lin_rec, gs["lin_slots"][:B], gs["lin_fresh"][:B])
        ctx = FwdCtx(positions=gs["pos"][:B], cu_seqlens=None, max_seqlen=1, kv=kv, tp=self.tp, ep=self.ep, tp_symm=self._symm(), fuse_add_norm=True)
        hidden = self.model.hidden_states(gs["tokens"][:B], ctx)
        logits = self._logits(hidden)
        ids, lp = ops.sample(logits, gs["u"][:B], sp.temperature, sp.top_k, sp.top_p, sp.min_p)
        gs["ids"][:B].copy_(ids)
        gs["lp"][:B].copy_(lp)

    def _graph_decode(self, plan: StepPlan):
        """One decode step for every running sequence through a captured CUDA graph.
        Inputs are written into persistent buffers (one pinned staging copy); the
        batch is padded to a bucket size with rows that write to a scratch slot."""
        gs = self._graph_state()
        seqs = plan.seqs
        B = len(seqs)
        Bg = min(b for b in self._BUCKETS if b >= B)
        bs = self.block_size
        st = gs["stage"]
        scratch_block = self.num_blocks          # one block past the allocator's range
        # plain Python lists, one tensor construction: per-element tensor writes would
        # cost more host time than the whole step takes on the GPU
        rows = [[0] * Bg, [0] * Bg, [scratch_block * bs] * Bg, [1] * Bg, [0] * Bg, [0] * Bg]
        owner, blen = gs["bt_owner"], gs["bt_len"]
        for i, s in enumerate(seqs):
            p = s.num_computed                   # position of the token fed now
            if s.inflight:
                # sampled by the step before, not read back yet: the device takes it from that step's output
                rows[4][i], rows[5][i] = s._row, 1
            else:
                rows[0][i] = s.output[-1] if s.output else s.prompt[-1]
            rows[1][i] = p + s.rope_delta        # rotary position (text after images is shifted)
            rows[2][i] = s.blocks[p // bs] * bs + p % bs
            rows[3][i] = p + 1
            nb = len(s.blocks)
            # the cached row is valid for this sequence *in this life*: a preempted sequence comes back with the
            # same object but other blocks, so the key carries its preemption count as well
            who = (s, s.preemptions)
            same = owner[i] is not None and owner[i] != "pad" and owner[i][0] is s and owner[i][1] == s.preemptions
            if not same or blen[i] != nb:
                first = blen[i] if (same and blen[i] < nb) else 0      # only the new tail of a known table
                gs["bt_host"][i, first:nb] = torch.tensor(s.blocks[first:nb], dtype=torch.int32)
                gs["bt"][i, first:nb].copy_(gs["bt_host"][i, first:nb], non_blocking=True)
                xfer.h2d_bytes += (nb - first) * 4
                owner[i], blen[i] = who, nb
        grouped = self._update_groups(gs, seqs, Bg)
        for i in range(B, Bg):
            if owner[i] != "pad":
                gs["bt_host"][i, 0] = scratch_block
                gs["bt"][i, :1].copy_(gs["bt_host"][i, :1], non_blocking=True)
                owner[i], blen[i] = "pad", 1
        if self.arch.layer_types is not None:
            scratch_slot = self.max_num_seqs + 1             # padded rows update a state nobody reads
            gs["lin_stage"][:Bg] = torch.tensor(self._state_slots_of(seqs) + [scratch_slot] * (Bg - B), dtype=torch.int64)
            gs["lin_slots"].copy_(gs["lin_stage"], non_blocking=True)
            xfer.h2d_bytes += gs["lin_stage"].numel() * 8
        st[:, :Bg] = torch.tensor(rows, dtype=torch.int64)
        gs["in64"].copy_(st, non_blocking=True)              # one pinned -> device copy per step
        gs["seq_lens"].copy_(gs["in64"][3])                   # int64 -> int32 on the device
        # input tokens: from the host where it knows them, else from the previous step's samples on the device
        # (outside the captured graph: a warm-up run of the body overwrites ``ids``)
        torch.where(gs["in64"][5] != 0, gs["ids"].index_select(0, gs["in64"][4]), gs["in64"][0], out=gs["tokens"])
        xfer.h2d_bytes += st.numel() * 8
        gs["u"][:Bg].copy_(torch.rand(Bg, device=self.device, generator=self.gen))
        sp = seqs[0].sampling
        key = (Bg, sp.key(), grouped)
        gs["use_groups"] = grouped
        if self._emulate_graphs:
            self._decode_body(Bg, sp)
            return gs["ids"][:B], gs["lp"][:B]
        g = self._graphs.get(key)
        if g is None:
            # warm-up on a side stream, then capture
            recurrent = self.arch.layer_types is not None
            if recurrent:
                # the warm-up run must not advance any sequence's recurrent state (the replay below does that
                # once): every row works on the scratch slot meanwhile
                gs["lin_slots"].fill_(self.max_num_seqs + 1)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._decode_body(Bg, sp)
            torch.cuda.current_stream().wait_stream(side)
            if recurrent:
                gs["lin_slots"].copy_(gs["lin_stage"], non_blocking=True)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._decode_body(Bg, sp)
            self._graphs[key] = g
        g.replay()
        return gs["ids"][:B], gs["lp"][:B]

    def _update_groups(self, gs, seqs, Bg: int) -> bool:
        """Which rows of the decode batch share their first KV blocks (prefix sharing gave the samples of a prompt the
        same physical blocks): the decode attention then reads those blocks once per group.  The tables only change
        when the batch does; they are rebuilt and uploaded then.  Returns whether any group exists."""
        if self.arch.use_mla or self.arch.layer_types is not None or not seqs:
            return False
        rep = self.arch.num_attention_heads // max(self.arch.num_key_value_heads, 1)
        if self.arch.head_dim != 128 or self.block_size != 64 or rep > 4 or os.environ.get("CLB200_GROUPED_DECODE", "1") == "0":
            return False
        sig = tuple((id(s), s.preemptions) for s in seqs)
        if gs["grp_key"] == (sig, Bg):
            return gs["grp_any"]
        by_first = {}
        for i, s in enumerate(seqs):
            if s.blocks:
                by_first.setdefault(s.blocks[0], []).append(i)
        G = max(Bg // 2, 1)
        st = gs["grp_stage"]
        st.zero_()
        gq = st[:G * 8].view(G, 8)
        gq.fill_(-1)
        gn, bstart = st[G * 8:G * 9], st[G * 9:G * 9 + Bg]
        g = 0
        for rows in by_first.values():
            for c in range(0, len(rows), 8):
                part = rows[c:c + 8]
                if len(part) < 2 or g >= G:
                    continue
                lists = [seqs[i].blocks for i in part]
                n = 0                                   # blocks common to all members, always leaving each its last one
                limit = min(len(b) for b in lists) - 1
                while n < limit and all(b[n] == lists[0][n] for b in lists):
                    n += 1
                if n == 0:
                    continue
                gq[g, :len(part)] = torch.tensor(part, dtype=torch.int32)
                gn[g] = n
                for i in part:
                    bstart[i] = n
                g += 1
        dev_view = G * 9 + Bg
        gs["grp_q"][:G].copy_(st[:G * 8].view(G, 8), non_blocking=True)
        gs["grp_nblk"][:G].copy_(gn, non_blocking=True)
        gs["blk_start"][:Bg].copy_(bstart, non_blocking=True)
        xfer.h2d_bytes += dev_view * 4
        gs["grp_key"], gs["grp_any"] = (sig, Bg), g > 0
        return g > 0

    def _can_graph(self, plan: StepPlan) -> bool:
        if not self.use_graphs or plan.is_prefill:
            return False
        if not self._emulate_graphs:
            if self.device.type != "cuda":
                return False
            if ops.get_mode() != "native" or self.model.dtype != torch.bfloat16:
                return False    # the PyTorch statements of the ops (also taken for fp32 weights) synchronise with the host
        if any(n != 1 for n in plan.q_lens) or len(plan.seqs) > self._BUCKETS[-1]:
            return False
        if self.lockstep is not None and self.lockstep.size > 1:
            return False
        sp0 = plan.seqs[0].sampling
        if sp0.has_penalty:
            return False
        k0 = sp0.key()
        return all(s.sampling is sp0 or s.sampling.key() == k0 for s in plan.seqs)

    # ------------------------------------------------------------------ pipelined decode
    # A captured decode step ends with the sampled tokens on the device.  The next step's inputs (positions, KV
    # slots, block tables) do not depend on their values, and its input tokens can be taken from the device, so
    # the next step is launched first and the previous step's tokens are read back while it runs: the host's
    # work per step (scheduling, staging, appending tokens, stop checks) overlaps the GPU instead of adding to it.
    # Stop conditions that depend on a token's value (EOS, stop tokens) are therefore seen one step late: the
    # sequence takes part in one more step whose token is dropped.  A sequence whose pending token is its last by
    # length is known in advance and left out of the next step.
    def _last_by_length(self, s: Sequence) -> bool:
        return len(s.output) + s.inflight >= s.max_new_tokens or s.length + s.inflight >= self.max_model_len

    def _start_readback(self, seqs, ids, lps):
        """Snapshot the step's samples and start their copy to pinned host memory; returns the pending record."""
        gs = self._gs
        par = gs["parity"]
        gs["parity"] = par ^ 1
        B = len(seqs)
        dev_buf, host_buf = gs["out_dev"][par], gs["out_host"][par]
        dev_buf[0, :B].copy_(ids)                      # token ids are exact in fp32: vocab < 2^24
        dev_buf[1, :B].copy_(lps)
        host_buf[:, :B].copy_(dev_buf[:, :B], non_blocking=True)
        if gs["out_event"][par] is not None:
            gs["out_event"][par].record()
        xfer.d2h_bytes += 2 * B * 4
        return {"seqs": list(seqs), "par": par}

    def _complete(self, pend, sched: Scheduler, eos_id):
        """Wait for a launched step's tokens, append them and apply the stop conditions."""
        gs = self._gs
        if gs["out_event"][pend["par"]] is not None:
            gs["out_event"][pend["par"]].synchronize()
        B = len(pend["seqs"])
        both = gs["out_host"][pend["par"]][:, :B].tolist()
        for s in pend["seqs"]:
            s.inflight = 0
        live = [(s, int(t), lp) for s, t, lp in zip(pend["seqs"], both[0], both[1]) if not s.finished]
        self._apply_tokens(sched, live, eos_id)

    def drain(self, sched: Scheduler, eos_id):
        """Read back the step that is still in flight, if any."""
        pend, self._pending = self._pending, None
        if pend is not None:
            self._complete(pend, sched, eos_id)

    def take_finished(self) -> List[Sequence]:
        out, self._finished_buf = self._finished_buf, []
        return out

    @torch.no_grad()
    def step(self, sched: Scheduler, plan: StepPlan, eos_id: Optional[int]):
        pend = self._pending
        if self._can_graph(plan):
            seqs = plan.seqs
            if pend is not None:
                # sequences whose token in flight is their last one do not decode again
                seqs = [s for s in seqs if not (s.inflight and self._last_by_length(s))]
            if seqs:
                part = plan if len(seqs) == len(plan.seqs) else StepPlan(seqs, [1] * len(seqs), False, [True] * len(seqs))
                ids, lps = self._graph_decode(part)
                for s in seqs:
                    s.num_computed += 1
                if not self.pipelined:
                    self._finish_step(sched, seqs, ids, lps, eos_id)
                    return
                new = self._start_readback(seqs, ids, lps)
                if pend is not None:
                    self._complete(pend, sched, eos_id)      # the previous step's tokens, while this one runs
                for i, s in enumerate(seqs):
                    s.inflight, s._row = 1, i
                self._pending = new
                return
            self.drain(sched, eos_id)
            return
        if pend is not None:
            # this step needs the host to know every token: finish the step in flight first and drop the
            # sequences that turn out to have ended with it
            self.drain(sched, eos_id)
            if any(s.finished for s in plan.seqs):
                keep = [i for i, s in enumerate(plan.seqs) if not s.finished]
                if not keep:
                    return
                plan = StepPlan([plan.seqs[i] for i in keep], [plan.q_lens[i] for i in keep], plan.is_prefill,
                                [plan.samples[i] for i in keep])
        tokens, ctx, last_rows = self._build_inputs(plan)
        x = None
        if self._embed_patch is not None:
            # image placeholder rows take the vision tower's embeddings
            from chatlearn_b200.models.nn.model import embed as _embed
            rows_, src_ = self._embed_patch
            x = _embed(self.model.block_by_name["embed"].params, tokens, ctx).to(self.model.dtype).clone()
            x.index_copy_(0, rows_, src_.to(x.dtype))
            self._embed_patch = None
        hidden = self.model.hidden_states(tokens, ctx, x=x)
        for s, n in zip(plan.seqs, plan.q_lens):
            s.num_computed += n
        rows = [i for i, smp in enumerate(plan.samples) if smp]
        if not rows:
            return
        sel = last_rows[torch.tensor(rows, device=self.device)] if len(rows) != len(plan.seqs) else last_rows
        logits = self._logits(hidden.index_select(0, sel))
        seqs = [plan.seqs[i] for i in rows]
        # group rows by sampling parameters (one kernel launch per distinct setting)
        groups: Dict[Any, List[int]] = {}
        for j, s in enumerate(seqs):
            groups.setdefault(s.sampling.key(), []).append(j)
        ids = torch.empty(len(seqs), dtype=torch.long, device=self.device)
        lps = torch.empty(len(seqs), dtype=torch.float32, device=self.device)
        u_all = torch.rand(len(seqs), device=self.device, generator=self.gen)
        for key, js in groups.items():
            sp = seqs[js[0]].sampling
            jj = torch.tensor(js, device=self.device)
            z = logits if len(js) == len(seqs) else logits.index_select(0, jj)
            if sp.has_penalty:
                V = z.shape[-1]
                counts = torch.zeros(len(js), V, dtype=torch.int32, device=self.device)
                pmask = torch.zeros(len(js), V, dtype=torch.bool, device=self.device)
                for r, j in enumerate(js):
                    if seqs[j].output:
                        o = torch.tensor(seqs[j].output, device=self.device)
                        counts[r].index_add_(0, o, torch.ones_like(o, dtype=torch.int32))
                    pmask[r, torch.tensor(seqs[j].prompt, device=self.device)] = True
                z = ops.apply_penalties(z, counts, sp.presence_penalty, sp.frequency_penalty,
                                        sp.repetition_penalty, pmask)
            i_, l_ = ops.sample(z, u_all if len(js) == len(seqs) else u_all.index_select(0, jj),
                                sp.temperature, sp.top_k, sp.top_p, sp.min_p)
            if len(js) == len(seqs):
                ids, lps = i_, l_
            else:
                ids[jj], lps[jj] = i_, l_
        self._finish_step(sched, seqs, ids, lps, eos_id)

    def _finish_step(self, sched: Scheduler, seqs, ids, lps, eos_id):
        """Read the sampled tokens back and apply the stop conditions."""
        # one device -> host read per step (token ids are exact in fp32: vocab < 2^24)
        both = xfer.tolist(torch.stack([ids.float(), lps.float()]))
        self._apply_tokens(sched, [(s, int(t), lp) for s, t, lp in zip(seqs, both[0], both[1])], eos_id)

    def _apply_tokens(self, sched: Scheduler, triples, eos_id):
        for s, tok, lp in triples:
            s.output.append(tok)
            s.logprobs.append(lp)
            sp = s.sampling
            if not sp.ignore_eos and (tok == eos_id or tok in sp.stop_token_ids):
                sched.finish(s, "stop")
            elif len(s.output) >= s.max_new_tokens or s.length >= self.max_model_len:
                sched.finish(s, "length")
            if s.finished:
                self._finished_buf.append(s)
                if self.arch.layer_types is not None:
                    slot = self._state_slot.pop(id(s), None)
                    if slot is not None:
                        self._free_state_slots.append(slot[0])

    @torch.no_grad()
    def _idle_step(self):
        """Forward of zero tokens: keeps this rank in the collectives of its peers."""
        dev = self.device
        z = lambda dt: torch.zeros(0, dtype=dt, device=dev)  # noqa: E731
        kv = KVCtx(self.k_cache, self.v_cache, z(torch.long), torch.zeros(0, 1, dtype=torch.int32, device=dev),
                   z(torch.int32), z(torch.int32), True, lin=self._linear_state([]))
        ctx = FwdCtx(positions=z(torch.long), cu_seqlens=torch.zeros(1, dtype=torch.int32, device=dev),
                     max_seqlen=0, kv=kv, tp=self.tp, ep=self.ep, tp_symm=self._symm(), fuse_add_norm=True)
        self.model.hidden_states(z(torch.long), ctx)

    # ------------------------------------------------------------------ public
    @torch.no_grad()
    def _attach_images(self, s: Sequence, mm: Dict[str, Any]):
        """Run the vision tower once for a request and remember where its embeddings go."""
        assert self.vision is not None, "this engine was built without a vision tower"
        from chatlearn_b200.models.nn.vision import mrope_positions
        grid = mm["image_grid_thw"]
        grid = grid.tolist() if torch.is_tensor(grid) else [list(g) for g in grid]
        px = torch.as_tensor(mm["pixel_values"]).to(self.device)
        embeds = self.vision(px, grid)
        taps = []
        if isinstance(embeds, tuple):            # towers with deep-stack taps (Qwen3-VL)
            embeds, taps = embeds
        embeds = embeds.to(self.model.dtype)
        itok, visual = self.arch.image_token_id, set(self.arch.visual_token_ids)
        # (a prompt that continues an earlier partial response may hold placeholder tokens the model generated
        # itself, after those of its images: they are ordinary tokens)
        where = [j for j, tkn in enumerate(s.prompt) if tkn in visual][:embeds.shape[0]]
        assert len(where) == embeds.shape[0], \
            f"{len(where)} image / video placeholder tokens in the prompt but {embeds.shape[0]} embeddings"
        pos3, delta = mrope_positions(torch.tensor(s.prompt), grid, itok, self.vision.arch.spatial_merge_size,
                                      self.arch.video_token_id, mm.get("visual_time_steps"))
        s.mm = {"embeds": embeds, "pos3": pos3, "ordinal": {j: o for o, j in enumerate(where)},
                "deepstack": [t.to(self.model.dtype) for t in taps]}
        s.rope_delta = int(delta)
        self._image_rows_seen = getattr(self, "_image_rows_seen", 0) + len(where)      # statistics

    def open_session(self, eos_id: Optional[int] = None) -> "RolloutSession":
        """A scheduler that stays open: requests are submitted and collected one by one while the engine keeps
        stepping (``generate`` is one session that is filled once and drained)."""
        return RolloutSession(self, eos_id)

    def generate(self, prompts: List[List[int]], sampling: Any, eos_id: Optional[int] = None,
                 max_new_tokens: Optional[List[int]] = None, mm_inputs: Optional[List[Optional[Dict]]] = None) -> List[Sequence]:
        """Generate for a batch of token-id prompts.  ``sampling`` is one
        ``SamplingParams`` or a list (one per prompt); ``max_new_tokens`` optionally
        overrides the per-request budget (partial rollout)."""
        sess = self.open_session(eos_id)
        seqs = []
        for i, p in enumerate(prompts):
            sp = sampling[i] if isinstance(sampling, (list, tuple)) else sampling
            seqs.append(sess.submit(p, sp, max_new_tokens[i] if max_new_tokens is not None else None,
                                    mm_inputs[i] if mm_inputs is not None else None))
        while sess.poll() is not None:
            pass
        sess.close()
        return seqs

    # ------------------------------------------------------------------ sleep / wake
    def offload(self, tags=(TAG_WEIGHTS, TAG_KV_CACHE)):
        if TAG_KV_CACHE in tags:
            self.free_kv_cache()

    def onload(self, tags=(TAG_WEIGHTS, TAG_KV_CACHE)):
        if TAG_KV_CACHE in tags:
            self.alloc_kv_cache()



class RolloutSession:
    """Per-request front of the engine: ``submit`` a request at any time, ``poll`` runs one scheduler step and
    returns the requests that finished in it.

    Parity: the reference's agent rollouts run one coroutine per request against an asynchronous SGLang engine
    (chatlearn/models/sglang_module.py:403-413 ``engine.async_generate``; chatlearn/models/agent/agent_module.py:
    82-100 ``generate_per_request``), so a trajectory's next turn starts as soon as its previous one ends,
    whatever the other requests are doing.  Here the same holds within one process: a request submitted between
    two steps joins the running batch at the next step (continuous batching), a finished one is handed back at
    once, and nothing waits for the slowest request of a "batch".  ``AsyncRollout`` puts asyncio futures on top.

    Under lock-step groups (replicas that share expert-parallel collectives) ``poll`` keeps a replica without
    work in its peers' collectives and reports the end (``None``) only when no replica has work left.
    """

    def __init__(self, engine: RolloutEngine, eos_id: Optional[int] = None):
        engine.alloc_kv_cache()
        self.engine = engine
        self.eos_id = engine.arch.eos_token_id if eos_id is None else eos_id
        # requests with the same prompt (the samples of a GRPO group) share the prompt's KV blocks; not with
        # recurrent layers, whose state is per sequence and cannot be adopted block-wise
        share = engine.arch.layer_types is None and os.environ.get("CLB200_PREFIX_SHARING", "1") != "0"
        self.sched = Scheduler(engine.num_blocks, engine.block_size, engine.max_num_seqs, engine.max_tokens,
                               prefix_sharing=share)
        self.tm = {"sched_s": 0.0, "prefill_s": 0.0, "decode_s": 0.0, "prefill_steps": 0, "decode_steps": 0}
        self._instant: List[Sequence] = []           # requests with no budget: finished on arrival
        self.submitted = 0

    def submit(self, prompt: List[int], sampling: "SamplingParams", max_new_tokens: Optional[int] = None,
               mm: Optional[Dict[str, Any]] = None) -> Sequence:
        eng = self.engine
        mx = sampling.max_tokens if max_new_tokens is None else max_new_tokens
        mx = max(0, min(mx, eng.max_model_len - len(prompt)))
        s = Sequence(eng._req_counter, list(prompt), mx, sampling)
        eng._req_counter += 1
        self.submitted += 1
        if mm is not None and mm.get("pixel_values") is not None and len(mm["image_grid_thw"]):
            eng._attach_images(s, mm)
        if mx == 0:
            s.finished, s.finish_reason = True, "length"
            self._instant.append(s)
        else:
            self.sched.add(s)
        return s

    def has_work(self) -> bool:
        return bool(self._instant) or self.sched.has_work()

    def poll(self) -> Optional[List[Sequence]]:
        """One engine step.  Returns the requests that finished in it (possibly none), or ``None`` when there is
        nothing left to do (on every replica of a lock-step group)."""
        eng, sched = self.engine, self.sched
        out, self._instant = self._instant, []
        busy = sched.has_work()
        if not busy and eng._pending is not None:
            eng.drain(sched, self.eos_id)                # the last step's tokens (all dropped or final)
            out.extend(eng.take_finished())
            busy = sched.has_work()
        lock = eng.lockstep is not None and eng.lockstep.size > 1
        if lock:
            import torch.distributed as dist
            flag = torch.tensor([1 if (busy or out) else 0], device=eng.device)
            eng.lockstep.all_reduce_(flag, op=dist.ReduceOp.MAX)
            if int(flag.item()) == 0:
                return None
            if not busy:
                eng._idle_step()
                return out
        elif not busy:
            return out if out else None
        t0 = time.perf_counter()
        plan = sched.schedule()
        t1 = time.perf_counter()
        self.tm["sched_s"] += t1 - t0
        if plan is None:
            if lock:
                eng._idle_step()
                return out
            return out if out else None
        eng.step(sched, plan, self.eos_id)           # ends with the read-back of the sampled tokens
        kind = "decode" if max(plan.q_lens) == 1 else "prefill"
        self.tm[kind + "_s"] += time.perf_counter() - t1
        self.tm[kind + "_steps"] += 1
        out.extend(eng.take_finished())
        return out

    def close(self):
        """Publish the session's statistics on the engine and check the peer-memory status words."""
        eng = self.engine
        eng.drain(self.sched, self.eos_id)
        eng.take_finished()
        eng.stats = dict(self.sched.stats)
        eng.stats.update(self.tm)
        if eng.ep_symm is not None:
            st = eng.ep_symm.status()
            if st:
                raise RuntimeError(
                    f"expert-parallel peer-memory dispatch reported status {st} "
                    "(1: a peer did not arrive within the wait limit, 2: an expert's receive region overflowed; "
                    "raise the capacity factor or set CLB200_SYMM_EP=0)")


class AsyncRollout:
    """asyncio front of a session: ``seq = await rollout.generate(prompt_ids, sampling)`` per request.

    One task drives the engine while any request is outstanding and yields to the event loop after every step,
    so the coroutine of a request that just finished can run its tools and submit its next turn before the
    next step is scheduled.  For a replica of one process (no tensor-parallel peers to keep in step)."""

    def __init__(self, engine: RolloutEngine, eos_id: Optional[int] = None):
        self.session = engine.open_session(eos_id)
        self._waiting: Dict[int, Any] = {}
        self._driver = None

    async def generate(self, prompt: List[int], sampling: "SamplingParams", max_new_tokens: Optional[int] = None,
                       mm: Optional[Dict[str, Any]] = None) -> Sequence:
        import asyncio
        loop = asyncio.get_running_loop()
        seq = self.session.submit(prompt, sampling, max_new_tokens, mm)
        fut = loop.create_future()
        self._waiting[seq.req_id] = fut
        if self._driver is None or self._driver.done():
            self._driver = loop.create_task(self._drive())
        return await fut

    async def _drive(self):
        import asyncio
        while self._waiting:
            try:
                done = self.session.poll()
            except BaseException as e:              # every waiter learns of a failed step
                for fut in self._waiting.values():
                    if not fut.done():
                        fut.set_exception(e)
                self._waiting.clear()
                raise
            if done is None:
                break
            for s in done:
                fut = self._waiting.pop(s.req_id, None)
                if fut is not None and not fut.done():
                    fut.set_result(s)
            await asyncio.sleep(0)

    def close(self):
        self.session.close()
