"""GRPO policy trainer / scorer on the tensor-, pipeline-, context- and
expert-parallel back end.

Parity: chatlearn/algorithm/grpo_utils/megatron_policy_trainer.py:55-327 and
megatron_utils/train_helper.py:233-603 (THD packing with every sequence padded for
CP, CP zig-zag split, per-token loss sums with the global token count, log-prob
re-gather over CP, last-pipeline-stage outputs).  What Megatron-Core provides in
the reference (TP layers, 1F1B schedule, alltoall MoE dispatcher, distributed
optimizer) is this framework's own: TP/EP-sharded ``CausalLM`` leaves with the
collectives in ``parallel.groups``, the vocab-parallel fused log-prob op, and the
pipeline schedule below over NCCL point-to-point.
"""
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from chatlearn_b200 import ops
from chatlearn_b200.models.megatron_module import MegatronModule
from chatlearn_b200.models.nn import FwdCtx
from chatlearn_b200.models.nn.model import decoder_layer
from chatlearn_b200.utils import xfer
from .trainer_utils import PackedBatch, pack_samples, split_microbatch, unpack_per_sample


class MegatronPolicyTrainer(MegatronModule):
    def setup(self):
        super().setup()
        self._metric_prefix = "policy_trainer" if self.trainable else self.name

    # ------------------------------------------------------------------ batching
    def _max_reduce(self, n: int) -> int:
        """Bin counts must agree on every rank that runs collectives together: the
        whole role when pipeline or expert parallelism couples the data-parallel
        ranks, else the model-parallel group."""
        t = torch.tensor([n], dtype=torch.int64, device=self.device)
        for g in (self.mp_group, self.ep_group, self.role_group):
            if g is not None and g.size > 1:
                g.all_reduce_(t, op=dist.ReduceOp.MAX)
        return int(t.item())

    def _microbatches(self, data_list: List[Dict], for_train: bool):
        ma = self.module_args
        if ma.packing:
            return split_microbatch(data_list, packing=True, max_train_token=ma.max_token_in_packing,
                                    max_reduce=self._max_reduce)
        mbs = ma.train_micro_batch_size if for_train else ma.generation_batch_size
        return split_microbatch(data_list, micro_batch_size=max(int(mbs), 1))

    def _prepare(self, mb: List[Dict]):
        """Packed row of a micro-batch, this CP rank's zig-zag slice and the context."""
        cp = self.cp_size
        mult = (2 * cp if cp > 1 else 1) * (self.tp_size if self.seq_parallel else 1)    # rows split evenly over cp, then tp
        batch = pack_samples(mb, seq_multiple=mult) if mb else None
        if batch is None:
            return None, None, None
        batch.to(self.device)
        ctx = FwdCtx(positions=batch.positions, cu_seqlens=batch.cu_seqlens, max_seqlen=batch.max_seqlen,
                     tp=self.tp_group if self.tp_size > 1 else None, ep=self.ep, seq_parallel=self.seq_parallel)
        local = None
        valid = batch.valid
        if cp > 1:
            plan = self.cp.plan(batch.seq_lens, self.device)
            local = plan["local"]
            ctx.cp, ctx.cp_plan = self.cp, plan
            ctx.positions = batch.positions.index_select(0, local)
            valid = valid.index_select(0, local) if valid is not None else None
        if valid is not None and self.seq_parallel and self.tp_size > 1:
            n = valid.shape[0] // self.tp_size                     # this tensor-parallel rank's rows
            valid = valid.narrow(0, self.tp_rank * n, n)
        ctx.row_valid = valid
        return batch, ctx, local

    # ------------------------------------------------------------------ pipeline plumbing
    def _send(self, t: torch.Tensor, to_stage: int):
        dist.send(t.contiguous(), self.pp_group.ranks[to_stage], group=self.pp_group.pg)

    def _exchange(self, send_t: torch.Tensor, to_stage: int, shape, dtype, from_stage: int) -> torch.Tensor:
        """Send one tensor and receive another with both transfers posted together."""
        out = torch.empty(tuple(shape), dtype=dtype, device=self.device)
        ops_ = [dist.P2POp(dist.isend, send_t.contiguous(), self.pp_group.ranks[to_stage], self.pp_group.pg),
                dist.P2POp(dist.irecv, out, self.pp_group.ranks[from_stage], self.pp_group.pg)]
        for req in dist.batch_isend_irecv(ops_):
            req.wait()
        return out

    def _recv(self, shape, dtype, from_stage: int) -> torch.Tensor:
        t = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(t, self.pp_group.ranks[from_stage], group=self.pp_group.pg)
        return t

    def _stage_forward(self, batch: PackedBatch, ctx: FwdCtx, local, x_in: Optional[torch.Tensor],
                       chunk: Optional[int] = None):
        """Forward of this pipeline stage (of its model chunk ``chunk`` under the interleaved schedule).  Returns
        hidden states, or ``(logprobs, entropy)`` where the model ends."""
        tokens = batch.tokens if local is None else batch.tokens.index_select(0, local)
        first = self.is_first_stage and (chunk is None or chunk == 0)
        last = self.is_last_stage and (chunk is None or chunk == self.vpp_size - 1)
        hook = None
        if torch.is_grad_enabled() and getattr(self.module_args, "recompute_granularity", None) == "full":
            from torch.utils.checkpoint import checkpoint
            arch = self.model.arch

            def hook(l, p, x, c):
                return checkpoint(lambda xx: decoder_layer(arch, p, xx, c, l), x, use_reentrant=False)
        x0 = None
        if getattr(self, "vision", None) is not None:
            from chatlearn_b200.models.nn.vision import multimodal_inputs
            # (image rows and positions are addressed in the whole packed row: under context and sequence parallelism
            # the inputs are built for the whole row and this rank keeps its slice)
            sp_rows, ctx.seq_parallel = ctx.seq_parallel and self.tp_size > 1, False
            x0 = multimodal_inputs(self.model, self.vision, batch.tokens, batch.seq_lens, batch.mm or [], ctx,
                                   with_embeddings=first)
            ctx.seq_parallel = sp_rows
            if local is not None:
                ctx.mrope_positions = ctx.mrope_positions.index_select(1, local)
                if x0 is not None:
                    x0 = x0.index_select(0, local)
                if ctx.deepstack is not None:
                    rows, taps = ctx.deepstack
                    where = torch.full((batch.tokens.shape[0],), -1, dtype=torch.long, device=rows.device)
                    where[local] = torch.arange(local.numel(), device=rows.device)
                    mine = where[rows]
                    keep = (mine >= 0).nonzero(as_tuple=True)[0]
                    ctx.deepstack = (mine[keep], [t.index_select(0, keep) for t in taps])
            if sp_rows:
                n = (batch.tokens.shape[0] if local is None else local.numel()) // self.tp_size
                if x0 is not None:
                    x0 = self.tp_group.scatter_seq(x0)           # (backward: the gradient rows of all ranks)
                if ctx.deepstack is not None:
                    rows, taps = ctx.deepstack
                    mine = rows - self.tp_rank * n
                    keep = ((mine >= 0) & (mine < n)).nonzero(as_tuple=True)[0]
                    ctx.deepstack = (mine[keep], [t.index_select(0, keep) for t in taps])
            if ctx.deepstack is not None:
                lo, hi = self.model.layer_range
                assert hi - lo >= len(ctx.deepstack[1]), "the first pipeline stage must hold every deep-stack layer"
        # embedding where the model starts, final norm where it ends (both decided inside by the layer range)
        h = self.model.hidden_states(tokens, ctx, hook, x=x0 if first else x_in, chunk=chunk)
        if not last:
            return h
        if ctx.seq_parallel:
            # the output head needs every row on every rank; its input gradient is already summed over the
            # vocabulary shards there, so the backward of this gather just keeps this rank's rows
            h = self.tp_group.gather_seq(h, 0)
        labels = batch.labels if local is None else batch.labels.index_select(0, local)
        w = self.model.lm_head_weight()
        if self.tp_size > 1 and w.shape[0] != self.model.arch.vocab_size:
            from chatlearn_b200.parallel.tp_ops import vocab_parallel_logprob_entropy
            return vocab_parallel_logprob_entropy(h, w, labels, self.tp_group)
        return ops.lmhead_logprob_entropy(h, w, labels)

    def _local_tokens(self, batch: PackedBatch, local) -> int:
        """Rows of the tensors that cross a stage boundary on this rank."""
        n = int(local.numel()) if local is not None else batch.num_tokens
        return n // self.tp_size if self.seq_parallel else n

    # ------------------------------------------------------------------ scoring
    @torch.no_grad()
    def forward_step(self, data_list: List[Dict], iteration: int = 0, **kwargs) -> List[Dict]:
        tag = "old_logprobs" if self.trainable else "ref_logprobs"
        H = self.model.arch.hidden_size
        for mb in self._microbatches(data_list, for_train=False):
            batch, ctx, local = self._prepare(mb)
            if batch is None:
                continue
            n_local = self._local_tokens(batch, local)
            if self.vpp_size > 1:
                # the model's chunks in order: chunk g lives on stage g % pp; the row travels round the stages
                # once per chunk of a stage (a scoring pass has no bubble to fill, so no interleaving here)
                P, out = self.pp_size, None
                for gchunk in range(P * self.vpp_size):
                    if gchunk % P != self.pp_rank:
                        continue
                    x_in = None if gchunk == 0 else self._recv((n_local, H), self.compute_dtype, (self.pp_rank - 1) % P)
                    out = self._stage_forward(batch, ctx, local, x_in, chunk=gchunk // P)
                    if gchunk < P * self.vpp_size - 1:
                        self._send(out, (self.pp_rank + 1) % P)
                if not self.is_last_stage:
                    continue
            else:
                x_in = None if self.is_first_stage else self._recv((n_local, H), self.compute_dtype, self.pp_rank - 1)
                out = self._stage_forward(batch, ctx, local, x_in)
                if not self.is_last_stage:
                    self._send(out, self.pp_rank + 1)
                    continue
            lp = out[0]
            if self.cp_size > 1:
                lp = self.cp.gather_tokens(lp, ctx.cp_plan)      # true all-gather, global order
            for s, v in zip(mb, unpack_per_sample(lp, batch, mb)):
                s[tag] = v
        return data_list

    # ------------------------------------------------------------------ training
    def _loss(self, batch: PackedBatch, local, lp, ent, inv_norm):
        ma = self.module_args
        sel = (lambda t: t if (t is None or local is None) else t.index_select(0, local))
        use_ref = ma.kl_coef != 0.0 and batch.ref_logprobs is not None
        need_ent = ma.entropy_coef != 0.0
        if ma.use_group_sequence_policy:
            # sequence means need every token of a sequence: gather log-probs over CP first
            lp_full = lp if self.cp_size == 1 else self.cp_group.gather_seq(lp, 0).index_select(0, self.cp.plan(
                batch.seq_lens, self.device)["inv"])
            loss_tok, cpos, cneg = ops.gspo_token_loss(
                lp_full, batch.old_logprobs, batch.advantages, batch.seq_ids, len(batch.seq_lens),
                batch.loss_mask, ma.pos_clip_ratio, ma.neg_clip_ratio, ma.diff_clip_ratio, ma.final_clip_ratio)
            m = batch.loss_mask
            # every CP rank evaluates the loss of the full row, and the backward of the gather hands each rank the
            # gradient of its own rows only: the sum over the ranks' rows is the full gradient, once
            total = (loss_tok * m).sum()
            stats = torch.stack([(loss_tok.detach() * m).sum(), torch.zeros((), device=self.device),
                                 torch.zeros((), device=self.device), (cpos.float() * m).sum(),
                                 (cneg.float() * m).sum(), m.sum()]) / max(self.cp_size, 1)
            return total * inv_norm, stats
        return ops.grpo_loss_fused(
            lp, sel(batch.old_logprobs), sel(batch.ref_logprobs) if use_ref else None, sel(batch.advantages),
            sel(batch.loss_mask), ent if need_ent else ent.detach(), ma.pos_clip_ratio, ma.neg_clip_ratio,
            ma.diff_clip_ratio, ma.final_clip_ratio, ma.kl_coef, ma.entropy_coef if need_ent else 0.0, inv_norm)

    def train_step(self, data_list: List[Dict], **kwargs):
        st = self.state
        H = self.model.arch.hidden_size
        n_tok = torch.tensor([float(sum(int(s["response_token_length"]) for s in data_list))],
                             dtype=torch.float32, device=self.device)
        # every rank of a model-parallel group holds the same samples: count them once
        n_tok /= (self.tp_size * self.cp_size * self.pp_size)
        self.mp_group.all_reduce_(n_tok)
        if self.mesh.groups["dp"].size > 1:
            self.mesh.groups["dp"].all_reduce_(n_tok)
        inv_norm = 1.0 / max(float(n_tok.item()), 1.0)
        st.zero_grad()
        stats = torch.zeros(6, dtype=torch.float32, device=self.device)
        mbs = [self._prepare(mb) for mb in self._microbatches(data_list, for_train=True)]
        mbs = [m for m in mbs if m[0] is not None]
        # schedule: one-forward-one-backward.  Stage r first runs (stages - r - 1) forwards, then
        # alternates a forward with the backward of its oldest micro-batch in flight, then drains;
        # at most (stages - r) micro-batches keep their activations on a stage instead of all of
        # them.  The stage boundary tensors travel over NCCL point-to-point; on every pair of
        # neighbours both sides issue "activation k, then gradient j" in the same order.
        from collections import deque
        in_flight = deque()

        prev, nxt = self.pp_rank - 1, self.pp_rank + 1
        first, last = self.is_first_stage, self.is_last_stage

        def compute_forward(batch, ctx, local, x_in, chunk=None, n_aux=0):
            nonlocal stats
            out = self._stage_forward(batch, ctx, local, x_in, chunk)
            ends = last and (chunk is None or chunk == self.vpp_size - 1)
            auxes = ctx.aux_losses[n_aux:]              # the router losses of this chunk's layers
            if ends:
                lp, ent = out
                loss, s = self._loss(batch, local, lp, ent, inv_norm)
                for aux in auxes:
                    loss = loss + aux * (batch.loss_mask.sum() * inv_norm)
                stats += s.detach()
                return loss, x_in, None, True
            # auxiliary (router) losses of intermediate stages are back-propagated locally
            aux = sum(auxes) * (batch.loss_mask.sum() * inv_norm) if auxes else None
            return out, x_in, aux, False

        def compute_backward(out, x_in, aux, ends, g):
            if ends:
                out.backward()
            elif aux is not None:
                torch.autograd.backward([out, aux], [g, torch.ones_like(aux)])
            else:
                out.backward(g)
            return x_in.grad if x_in is not None else None

        def in_shape(k):
            return (self._local_tokens(mbs[k][0], mbs[k][2]), H)

        if self.vpp_size > 1:
            self._run_interleaved(mbs, compute_forward, compute_backward, in_shape)
            return self._finish_train_step(st, stats)
        n_mb = len(mbs)
        warm = min(self.pp_size - self.pp_rank - 1, n_mb)
        steady = n_mb - warm
        # warm-up: forwards only
        for k in range(warm):
            x_in = None if first else self._recv(in_shape(k), self.compute_dtype, prev).requires_grad_(True)
            item = compute_forward(*mbs[k], x_in)
            if not last:
                self._send(item[0].detach(), nxt)
            in_flight.append(item)
        # steady state: the activation of the new micro-batch and the gradient of the oldest one cross
        # a stage boundary in ONE exchange (both directions posted together), so neighbours never
        # wait on each other's sends
        x_in = None
        if steady > 0 and not first:
            x_in = self._recv(in_shape(warm), self.compute_dtype, prev).requires_grad_(True)
        for t in range(steady):
            k = warm + t
            item = compute_forward(*mbs[k], x_in)
            in_flight.append(item)
            old = in_flight.popleft()
            g = None
            if not last:
                g = self._exchange(item[0].detach(), nxt, old[0].shape, old[0].dtype, nxt)
            dx = compute_backward(*old, g)
            if t + 1 < steady:
                x_in = None if first else \
                    self._exchange(dx, prev, in_shape(k + 1), self.compute_dtype, prev).requires_grad_(True)
            elif not first:
                self._send(dx, prev)
        # cool-down: backwards only
        while in_flight:
            old = in_flight.popleft()
            g = None if last else self._recv(old[0].shape, old[0].dtype, nxt)
            dx = compute_backward(*old, g)
            if not first:
                self._send(dx, prev)
        return self._finish_train_step(st, stats)

    # ------------------------------------------------------------------ interleaved (virtual pipeline) schedule
    @staticmethod
    def interleaved_order(P: int, V: int, m: int, r: int):
        """Units of stage ``r`` in execution order, ``("F" | "B", micro-batch, chunk)``: Megatron's interleaved
        one-forward-one-backward order.  Micro-batches advance in groups of ``P``; a stage runs the group through
        its chunk 0, then through chunk 1, ...; backwards visit the chunks in reverse.  ``(P - r - 1) * 2 +
        (V - 1) * P`` forwards run before the first backward."""
        def unit(k, back):
            group, idx = divmod(k, P * V)
            width = min(P, m - group * P)              # the last group may hold fewer micro-batches
            if width < P:
                j, i = divmod(k - group * P * V, width)
            else:
                j, i = divmod(idx, P)
            return (group * P + i, (V - 1 - j) if back else j)
        total = m * V
        warm = min((P - r - 1) * 2 + (V - 1) * P, total)
        order = [("F",) + unit(k, False) for k in range(warm)]
        for i in range(total - warm):
            order.append(("F",) + unit(warm + i, False))
            order.append(("B",) + unit(i, True))
        order += [("B",) + unit(i, True) for i in range(total - warm, total)]
        return order

    @staticmethod
    def interleaved_ticks(P: int, V: int, m: int):
        """Global time table of the interleaved schedule: ``ticks[r][t]`` is the unit stage ``r`` runs at tick ``t``
        (or None).  A unit runs at the first tick after its input exists: the forward of chunk g needs the forward
        of chunk g - 1 of the same micro-batch (sent at the end of the tick it ran in), the backward of chunk g the
        backward of chunk g + 1 (or, for the last chunk, its own forward).  Every stage derives the same table, so
        at every tick a stage knows what its neighbours send it."""
        G = P * V

        def simulate(orders):
            done = {}                                          # (kind, mb, global chunk) -> tick
            at = [0] * P
            ticks = [[] for _ in range(P)]
            t = 0
            while any(at[r] < len(orders[r]) for r in range(P)):
                ran = []
                for r in range(P):
                    u = None
                    if at[r] < len(orders[r]):
                        kind, mb, j = orders[r][at[r]]
                        g = j * P + r
                        if kind == "F":
                            dep = None if g == 0 else ("F", mb, g - 1)
                        else:
                            dep = ("F", mb, g) if g == G - 1 else ("B", mb, g + 1)
                        if dep is None or done.get(dep, t) < t:
                            u = (kind, mb, j)
                            ran.append((kind, mb, g))
                            at[r] += 1
                    ticks[r].append(u)
                if not ran:
                    return None                                # every stage waits for another: not a valid order
                for key in ran:
                    done[key] = t
                t += 1
            return ticks

        ticks = simulate([MegatronPolicyTrainer.interleaved_order(P, V, m, r) for r in range(P)])
        if ticks is None:
            # always valid: every forward (chunk by chunk), then every backward
            fwd = [[("F", k, j) for j in range(V) for k in range(m)] for _ in range(P)]
            bwd = [[("B", k, j) for j in reversed(range(V)) for k in range(m)] for _ in range(P)]
            ticks = simulate([f + b for f, b in zip(fwd, bwd)])
        assert ticks is not None
        return ticks

    def _run_interleaved(self, mbs, compute_forward, compute_backward, in_shape):
        """Interleaved one-forward-one-backward over ``vpp_size`` model chunks per stage.  All stages walk the same
        global time table; what a tick's units produce crosses the stage boundaries in ONE batched exchange at the
        end of that tick (a stage posts the receive for a neighbour's output in the tick the neighbour produces
        it), so sends and receives always meet inside the same exchange."""
        P, V, r = self.pp_size, self.vpp_size, self.pp_rank
        G = P * V
        ticks = self.interleaved_ticks(P, V, len(mbs))
        nxt, prv = (r + 1) % P, (r - 1) % P
        acts, grads, saved = {}, {}, {}                        # inputs that arrived, by (micro-batch, chunk)
        for t in range(len(ticks[r])):
            u = ticks[r][t]
            send = []
            if u is not None:
                kind, k, j = u
                g = j * P + r
                if kind == "F":
                    x_in = None
                    if g > 0:
                        x_in = acts.pop((k, j)).requires_grad_(True)
                    ctx = mbs[k][1]
                    n_aux = len(ctx.aux_losses)
                    item = compute_forward(mbs[k][0], ctx, mbs[k][2], x_in, j, n_aux)
                    saved[(k, j)] = item
                    if g < G - 1:
                        send.append((item[0].detach(), nxt))
                else:
                    item = saved.pop((k, j))
                    dx = compute_backward(*item, None if g == G - 1 else grads.pop((k, j)))
                    if g > 0:
                        send.append((dx, prv))
            recv = []
            for peer, want in ((prv, "F"), (nxt, "B")):
                pu = ticks[peer][t] if t < len(ticks[peer]) else None
                if pu is None or pu[0] != want:
                    continue
                pg = pu[2] * P + peer
                if want == "F" and pg < G - 1:                 # its output is the input of my chunk pg + 1
                    recv.append((acts, (pu[1], (pg + 1) // P), peer))
                elif want == "B" and pg > 0:                   # its input gradient belongs to my chunk pg - 1
                    recv.append((grads, (pu[1], (pg - 1) // P), peer))
            if not send and not recv:
                continue
            ops_ = [dist.P2POp(dist.isend, x.contiguous(), self.pp_group.ranks[to], self.pp_group.pg) for x, to in send]
            for store, key, peer in recv:
                buf = torch.empty(in_shape(key[0]), dtype=self.compute_dtype, device=self.device)
                store[key] = buf
                ops_.append(dist.P2POp(dist.irecv, buf, self.pp_group.ranks[peer], self.pp_group.pg))
            for req in dist.batch_isend_irecv(ops_):
                req.wait()
        assert not acts and not grads and not saved

    def _sum_tied_embedding_grads(self, st):
        """Tied input / output embeddings under pipeline parallelism: the first stage holds the matrix for the
        look-up, the last stage a copy for the output head.  Their gradients are exchanged and added, so both copies
        take the same step (the reference leaves this to Megatron's embedding-gradient all-reduce between the two
        stages)."""
        if self.pp_size == 1 or not self.model.arch.tie_word_embeddings or not (self.is_first_stage or self.is_last_stage):
            return
        s = next(x for x in st.states if x.block.name == "embed")
        other = self.pp_size - 1 if self.is_first_stage else 0
        s.grad.add_(self._exchange(s.grad, other, s.grad.shape, s.grad.dtype, other))

    def _finish_train_step(self, st, stats):
        self._sum_tied_embedding_grads(st)
        grad_norm = st.step()
        # metrics live on the last stage; share them with the whole model-parallel group
        if self.pp_size > 1:
            self.pp_group.all_reduce_(stats)
        if self.mesh.groups["dp"].size > 1:
            self.mesh.groups["dp"].all_reduce_(stats)
        if self.cp_size > 1:
            self.cp_group.all_reduce_(stats)
        host = xfer.tolist(torch.cat([stats, grad_norm.reshape(1).float()]))
        n = max(host[5], 1.0)
        self._metric_list.append({
            "pg_loss": host[0] / n, "kl_loss": host[1] / n, "entropy_loss": host[2] / n, "grad_norm": host[6],
            "clip_pos_frac": host[3] / n, "clip_neg_frac": host[4] / n, "train_tokens": n})
        self._train_iteration += 1
