"""Parameter-sharded training state (FSDP2 semantics) over flat parameter blocks.

The reference shards every decoder layer's parameters with torch ``fully_shard``:
bf16 parameters are all-gathered before a layer's forward and again before its
backward, gradients are reduce-scattered right after the layer's backward, and
only 1/dp of parameters, gradients and optimizer state stay resident
(chatlearn/models/fsdp_module.py:356-394, ``reshard_after_forward``).  This is
the same contract on this package's blocks:

* resident per block: this rank's 1/dp slice of the compute-dtype parameters, of
  the fp32 master weights and Adam moments, and of the fp32 gradient accumulator;
* a *segment* (embedding, one decoder layer, head) runs inside one autograd
  function: its forward gathers the block into one of two pooled buffers, runs
  without a tape and keeps only the segment's input; its backward gathers the block
  again, re-runs the segment with a tape, back-propagates, reduce-scatters the
  block's fp32 gradient into the resident accumulator and releases the buffers.
  Activation recomputation and parameter re-gathering are therefore one mechanism;
* the gather of the next segment (previous one in backward) is issued on a side
  stream while the current one computes, and the reduce-scatter of a segment's
  gradient runs on that stream behind the next segment's backward.

With symmetric memory (one process per GPU over NVLink) the gather is a *pull*:
the parameter slices of all blocks live in one symmetric arena, they only change
at the optimizer step, so between steps every rank reads its peers' slices with
plain loads (the descriptor-table copy kernel of the weight synchronizer) whenever
it needs them: no rendezvous, no collective launch on the peers.  The gradient
reduce-scatter is the pull-and-sum kernel of ``symm_collectives`` (each rank reads
its slice of every peer's gradient buffer).  Without symmetric memory (CPU ranks,
gloo; ``CLB200_SYMM_FSDP=0``) both run as process-group collectives.
"""
import os
from typing import Dict, List, Optional, Sequence

import torch

from chatlearn_b200 import ops
from chatlearn_b200.models.nn.model import CausalLM, decoder_layer, embed, flush_pending
from .groups import Group
from .zero import BlockState, ShardedTrainState


class ReshardedTrainState(ShardedTrainState):
    """``ShardedTrainState`` whose compute-dtype parameters are sharded as well."""

    reshard = True

    def __init__(self, model: CausalLM, dp_group: Optional[Group] = None, **kw):
        kw.pop("grad_dtype", None)
        super().__init__(model, dp_group, grad_dtype=torch.float32, **kw)
        assert self.tp_size == 1 and self.edp is self.dp, "parameter sharding runs on the data-parallel group only"
        dev = model.device
        self.comm = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        self.order: List[str] = []                       # segment order of the last forward (for prefetching)
        self._pos: Dict[str, int] = {}
        self.by_name: Dict[str, BlockState] = {s.block.name: s for s in self.states}
        total = sum(s.shard_numel for s in self.states)
        self.max_numel = max(s.block.numel for s in self.states)
        # ---- resident slices: one arena of parameter slices (symmetric memory where there is any)
        self.symm_gather = None
        arena = None
        if (dev.type == "cuda" and self.dp.size > 1 and os.environ.get("CLB200_SYMM_FSDP", "1") != "0"
                and ops.get_mode() == "native"):
            from . import symm_collectives, symm_mem
            sg = symm_collectives.get(self.dp)
            if sg is not None:
                arena = symm_mem.empty(total, model.dtype, dev, group=self.dp.pg)
                self.symm_gather = sg
        if arena is None:
            arena = torch.empty(total, dtype=model.dtype, device=dev)
        self.param_arena = arena
        off = 0
        for s in self.states:
            s.arena_off = off
            s.param_shard = arena[off:off + s.shard_numel]
            s.param_shard.copy_(s.block.flat[s.lo:s.hi])
            off += s.shard_numel
            # the whole-block gradient buffer of the replicated mode is not kept
            s.grad = None
            s.grad_shard = torch.zeros(s.shard_numel, dtype=torch.float32, device=dev)
            self._unbind(s)
        # ---- pooled transient buffers: two whole-block parameter buffers, two whole-block fp32 gradient buffers
        self._pbuf = [torch.empty(self.max_numel, dtype=model.dtype, device=dev) for _ in range(2)]
        if self.symm_gather is not None:
            from . import symm_mem
            self._gbuf = [symm_mem.empty(self.max_numel, torch.float32, dev, group=self.dp.pg) for _ in range(2)]
        else:
            self._gbuf = [torch.empty(self.max_numel, dtype=torch.float32, device=dev) for _ in range(2)]
        self._pbuf_free_ev = [None, None]      # compute-stream event: the buffer's last user has finished
        self._gbuf_free_ev = [None, None]      # comm-stream event: the buffer's reduce-scatter has finished
        self._held: Dict[str, dict] = {}       # block name -> {"p": index, "g": index or None, "ready": event}
        self._flip_p = self._flip_g = 0
        self._tmp_shard = torch.empty(max(s.shard_numel for s in self.states), dtype=torch.float32, device=dev) \
            if self.symm_gather is not None else None
        self._pull_tables: Dict[str, tuple] = {}
        self._anchor = None
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        self.dp.barrier()

    # ------------------------------------------------------------------ plumbing
    @staticmethod
    def _unbind(s: BlockState):
        b = s.block
        b.flat = None
        for p in b.params.values():
            p.data = torch.empty(0, dtype=b.dtype, device=b.device)
            p.grad = None
            if hasattr(p, "main_grad"):
                p.main_grad = None

    def enable_symm(self) -> bool:
        return False        # the replicated mode's fused optimizer collectives do not apply: nothing is all-gathered at the step

    def _stream(self):
        return torch.cuda.stream(self.comm) if self.comm is not None else _Null()

    def _pull_table(self, s: BlockState, dst: torch.Tensor):
        """Descriptor table for the pull all-gather of one block into ``dst``: one contiguous row per rank,
        read from that rank's slice of the symmetric arena."""
        import numpy as np
        from chatlearn_b200.parallel import symm_mem
        from chatlearn_b200.synchronizer.kernel_executor import _DESC, _DTYPE_CODE
        key = (s.block.name, dst.data_ptr())
        hit = self._pull_tables.get(key)
        if hit is not None:
            return hit
        from chatlearn_b200.ops import native
        tile = native.C.weight_sync_tile_elems()
        esz = dst.element_size()
        arr = np.zeros(self.dp.size, dtype=_DESC)
        tiles = 0
        for r in range(self.dp.size):
            src = symm_mem.peer_pointer(self.param_arena, self.dp.ranks[r]) + s.arena_off * esz
            tpr = (s.shard_numel + tile - 1) // tile
            arr[r] = (src, dst.data_ptr() + r * s.shard_numel * esz, s.shard_numel, s.shard_numel, 1, s.shard_numel, tiles, tpr)
            tiles += tpr
        table = torch.from_numpy(arr.view(np.uint8).copy()).to(dst.device)
        code = _DTYPE_CODE[dst.dtype]
        hit = (table, self.dp.size, tiles, code, code)
        self._pull_tables[key] = hit
        return hit

    def _issue_gather(self, name: str):
        """Start gathering block ``name`` into a pooled buffer on the side stream."""
        if name in self._held:
            return
        s = self.by_name[name]
        i = self._flip_p
        self._flip_p ^= 1
        assert all(h["p"] != i for h in self._held.values()), "both pooled parameter buffers are in use"
        buf = self._pbuf[i][:s.block.numel]
        with self._stream():
            if self.comm is not None:
                if self._pbuf_free_ev[i] is not None:
                    self.comm.wait_event(self._pbuf_free_ev[i])
            if self.symm_gather is not None:
                from chatlearn_b200.ops import native
                native.weight_sync_run(*self._pull_table(s, buf))
            else:
                self.dp.all_gather_flat(buf, s.param_shard)
            ev = None
            if self.comm is not None:
                ev = torch.cuda.Event()
                ev.record(self.comm)
        self._held[name] = {"p": i, "g": None, "ready": ev}

    def gather(self, names: Sequence[str], with_grad: bool = False, prefetch: Optional[str] = None):
        """Bind the parameters of ``names`` to gathered buffers (waiting for a prefetch where one is in flight);
        with ``with_grad`` their leaves accumulate into a zeroed whole-block fp32 gradient buffer."""
        for n in names:
            self._issue_gather(n)
        for n in names:
            h, s = self._held[n], self.by_name[n]
            if h["ready"] is not None:
                torch.cuda.current_stream().wait_event(h["ready"])
                h["ready"] = None
            s.block.bind(self._pbuf[h["p"]][:s.block.numel])
            if with_grad:
                j = self._flip_g
                self._flip_g ^= 1
                if self.comm is not None and self._gbuf_free_ev[j] is not None:
                    torch.cuda.current_stream().wait_event(self._gbuf_free_ev[j])
                g = self._gbuf[j][:s.block.numel]
                g.zero_()
                s.block.enable_grad(g)
                h["g"] = j
        if prefetch is not None and len(self._held) < 2:
            self._issue_gather(prefetch)

    def release(self, names: Sequence[str], reduce_grads: bool = False):
        """Unbind the blocks; with ``reduce_grads`` their gradient buffers are reduce-scattered into the
        resident accumulators first (on the side stream, behind the compute that produced them)."""
        for n in names:
            h, s = self._held.pop(n), self.by_name[n]
            if reduce_grads and h["g"] is not None:
                j = h["g"]
                g = self._gbuf[j][:s.block.numel]
                if self.comm is not None:
                    done = torch.cuda.Event()
                    done.record()                                  # the segment's backward, on the compute stream
                    self.comm.wait_event(done)
                with self._stream():
                    if self.symm_gather is not None:
                        tmp = self._tmp_shard[:s.shard_numel]
                        self.symm_gather.reduce_scatter_pull(g, tmp, s.lo)
                        s.grad_shard.add_(tmp)
                    elif self.dp.size == 1:
                        s.grad_shard.add_(g)
                    else:
                        tmp = torch.empty(s.shard_numel, dtype=torch.float32, device=g.device)
                        self.dp.reduce_scatter_flat(tmp, g)
                        s.grad_shard.add_(tmp)
                    if self.comm is not None:
                        ev = torch.cuda.Event()
                        ev.record(self.comm)
                        self._gbuf_free_ev[j] = ev
            if self.comm is not None:
                ev = torch.cuda.Event()
                ev.record()
                self._pbuf_free_ev[h["p"]] = ev
            self._unbind(s)

    def _segment_names(self, key: str) -> List[str]:
        names = [key] + ([key + ".experts"] if key + ".experts" in self.by_name else [])
        if key == "head" and self.model.arch.tie_word_embeddings:
            names.append("embed")
        return names

    @torch.no_grad()
    def join_empty_microbatch(self):
        """A rank whose micro-batch list is shorter than its peers' still has to take part in the collectives
        of their forward and backward passes.  Pull gathers need no partner, so with symmetric memory only the
        reduce-scatters are joined (with zeros, last segment first); with process-group collectives the whole
        sequence of gathers and reduce-scatters of one micro-batch is replayed, prefetches included, because
        collectives must be issued in the same order on every rank."""
        if self.dp.size == 1:
            return
        assert self.order, "the first micro-batch of a rank must not be empty (the segment order is learned from it)"
        if self.symm_gather is None:
            for key in self.order:
                names = self._segment_names(key)
                self.gather(names, prefetch=self._neighbour(key, +1))
                self.release(names)
        for key in reversed(self.order):
            names = self._segment_names(key)
            self.gather(names, with_grad=True, prefetch=self._neighbour(key, -1))
            self.release(names, reduce_grads=True)

    # ------------------------------------------------------------------ optimizer step
    def zero_grad(self):
        for s in self.states:
            s.grad_shard.zero_()

    @torch.no_grad()
    def reduce_grads(self):
        # every segment's gradient was reduce-scattered right after its backward; wait for the last ones
        if self.comm is not None:
            torch.cuda.current_stream().wait_stream(self.comm)
        if self.replica is not None:
            # hybrid sharding: the other shard groups hold the same shards of their own samples' gradients
            for s in self.states:
                self.replica.all_reduce_(s.grad_shard)

    @torch.no_grad()
    def step(self, lr: Optional[float] = None):
        self.reduce_grads()
        norm = self.grad_norm()
        self.last_grad_norm = norm
        scale = 1.0
        if self.clip and self.clip > 0:
            scale = torch.clamp(self.clip / (norm + 1e-6), max=1.0)
        self.step_count += 1
        lr = self.lr if lr is None else lr
        for s in self.states:
            ops.adamw_step(s.master, s.grad_shard, s.exp_avg, s.exp_avg_sq, s.param_shard, self.step_count, lr,
                           self.betas[0], self.betas[1], self.eps, self.wd, scale)
        self._publish()
        return norm

    def _publish(self):
        """The new slices must be visible to every peer before anybody pulls them again."""
        if self.symm_gather is not None:
            torch.cuda.current_stream().synchronize()
            self.dp.barrier()

    @torch.no_grad()
    def rebuild_params(self):
        for s in self.states:
            if s.master is not None:
                s.param_shard.copy_(s.master)
        self._publish()

    def tensors_for(self, tag: str):
        out = []
        for s in self.states:
            if tag == "weights" and self.symm_gather is None:
                out.append((s, "param_shard"))
            elif tag == "grads":
                out.append((s, "grad_shard"))
            elif tag == "optimizer":
                out.extend([(s, "master"), (s, "exp_avg"), (s, "exp_avg_sq")])
        return out

    @torch.no_grad()
    def load_state_dict(self, sd: Dict):
        self.step_count = sd["step"]
        for s in self.states:
            b = sd["blocks"][s.block.name]
            assert (b["lo"], b["hi"]) == (s.lo, s.hi), "checkpoint was written with another dp size"
            s.master.copy_(b["master"])
            s.exp_avg.copy_(b["exp_avg"])
            s.exp_avg_sq.copy_(b["exp_avg_sq"])
            s.param_shard.copy_(s.master)
        self._publish()

    # ------------------------------------------------------------------ whole-model access (export, checkpoints)
    class _AllGathered:
        def __init__(self, st):
            self.st = st

        def __enter__(self):
            st = self.st
            for s in st.states:
                full = torch.empty(s.block.numel, dtype=s.block.dtype, device=s.param_shard.device)
                st.dp.all_gather_flat(full, s.param_shard)
                s.block.bind(full)
            return st.model

        def __exit__(self, *exc):
            for s in self.st.states:
                ReshardedTrainState._unbind(s)

    def all_gathered(self):
        """Context manager: every block whole and bound (HF export); collective over the data-parallel group."""
        return ReshardedTrainState._AllGathered(self)

    # ------------------------------------------------------------------ running the model
    def _seg(self, names: List[str], run, inputs, grad: bool):
        key = names[0]
        if key not in self._pos:
            self._pos[key] = len(self.order)
            self.order.append(key)
        if grad:
            # the parameters are not inputs of the function (they are bound inside it), so a scalar that
            # requires a gradient rides along: it makes autograd record the segment even when its real inputs
            # are integer tokens
            if self._anchor is None:
                self._anchor = torch.zeros((), device=self.model.device, requires_grad=True)
            return _Segment.apply(run, self, tuple(names), self._anchor, *inputs)
        nxt = self._neighbour(key, +1)
        self.gather(names, prefetch=nxt)
        out = run(*inputs)
        self.release(names)
        return out

    def _neighbour(self, key: str, step: int) -> Optional[str]:
        i = self._pos.get(key)
        if i is None:
            return None
        j = i + step
        return self.order[j] if 0 <= j < len(self.order) else None

    def logprobs(self, tokens, labels, ctx, temperature: float = 1.0, x=None, embed_fn=None):
        """``CausalLM.logprobs`` with every block gathered only while its segment runs.  ``embed_fn(tokens)``
        replaces the plain embedding look-up (vision-language rows: the tower's output goes into the image rows; it
        runs inside the first segment, with the embedding block and, if it is trained, the tower's block gathered)."""
        m = self.model
        arch = m.arch
        grad = torch.is_grad_enabled()
        self._fwd_ctx = ctx                # (the segments' backward passes find the auxiliary-loss weight here)
        if x is None:
            first = ["embed"] + (["vision"] if embed_fn is not None and "vision" in self.by_name else [])
            fn = embed_fn if embed_fn is not None else (lambda t: embed(m.block_by_name["embed"].params, t, ctx))

            def run_embed(t):
                # deep-stack taps of a vision tower leave the segment as outputs (and enter their layers' segments
                # as inputs), so that a trained tower receives their gradients across the segment boundaries
                ctx.deepstack = None
                h = _as(m.dtype, fn(t))
                return (h,) + tuple(ctx.deepstack[1]) if ctx.deepstack is not None else h
            x = self._seg(first, run_embed, (tokens,), grad)
        taps = ()
        if isinstance(x, (tuple, list)):
            x, taps = x[0], tuple(x[1:])
        for l in range(*m.layer_range):
            names = [f"layer{l}"] + ([f"layer{l}.experts"] if f"layer{l}.experts" in m.block_by_name else [])
            def run_layer(xx, tap=None, l=l):
                xx = decoder_layer(arch, m.layer_params(l), xx, ctx, l)
                if tap is None and ctx.deepstack is not None and l < len(ctx.deepstack[1]):
                    tap = ctx.deepstack[1][l]
                if tap is not None:
                    # vision features of tap l join the residual stream at the image rows (Qwen3-VL)
                    xx = xx.index_add(0, ctx.deepstack[0], tap.to(xx.dtype))
                return xx
            x = self._seg(names, run_layer, (x, taps[l]) if l < len(taps) else (x,), grad)
        head = ["head"] + (["embed"] if arch.tie_word_embeddings else [])

        def run_head(h, lab):
            if ctx.pending is not None:
                # inference passes fuse every residual add into the next norm: the last layer's MLP output is
                # still pending in the context and joins the stream here, inside the final norm
                h = flush_pending(h, ctx, m.final_norm_weight(), arch.rms_norm_eps)
            else:
                h = ops.rmsnorm(h, m.final_norm_weight(), arch.rms_norm_eps)
            return ops.lmhead_logprob_entropy(h, m.lm_head_weight(), lab, temperature)
        return self._seg(head, run_head, (x, labels), grad)


def _as(dtype, t):
    return t if t.dtype == dtype else t.to(dtype)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class _Segment(torch.autograd.Function):
    """One segment of the model under parameter sharding: gather → run without a tape → release in forward;
    gather → re-run with a tape → back-propagate → reduce-scatter the gradients → release in backward."""

    @staticmethod
    def forward(ctx, run, state: ReshardedTrainState, names, _anchor, *inputs):
        ctx.run, ctx.state, ctx.names = run, state, names
        with torch.no_grad():
            state.gather(names, prefetch=state._neighbour(names[0], +1))
            out = run(*inputs)
            state.release(names)
        ctx.save_for_backward(*inputs)
        return out

    @staticmethod
    def backward(ctx, *grads):
        state, names = ctx.state, ctx.names
        inputs = [t.detach().requires_grad_(t.is_floating_point()) for t in ctx.saved_tensors]
        state.gather(names, with_grad=True, prefetch=state._neighbour(names[0], -1))
        fc = getattr(state, "_fwd_ctx", None)
        n_aux = len(fc.aux_losses) if fc is not None else 0
        with torch.enable_grad():
            out = ctx.run(*inputs)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and o.requires_grad]
        if fc is not None and len(fc.aux_losses) > n_aux:
            # auxiliary (router balancing) losses of this segment: the forward ran without a tape, so they are
            # back-propagated here, from the re-run, with their weight in the objective
            aux, w = fc.aux_losses[n_aux:], fc.aux_weight
            del fc.aux_losses[n_aux:]
            if w is not None:
                pairs += [(a, torch.as_tensor(w, dtype=a.dtype, device=a.device)) for a in aux if a.requires_grad]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        state.release(names, reduce_grads=True)
        return (None, None, None, None) + tuple(t.grad if t.requires_grad else None for t in inputs)
