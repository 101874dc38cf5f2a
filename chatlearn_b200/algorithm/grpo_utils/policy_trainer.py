"""GRPO policy trainer / log-prob scorer on the FSDP-style back end.

Parity: chatlearn/algorithm/grpo_utils/policy_trainer.py:80-365.  Same contract:
``forward_step`` adds per-token ``old_logprobs`` / ``ref_logprobs`` to each sample;
``train_step`` runs one optimizer step over a mini-batch (micro-batching or
sequence packing, optional Ulysses split, GRPO clipped-ratio loss + k3 KL +
entropy bonus, global-token-mean normalisation, grad-norm clip, AdamW) and
records ``pg_loss, kl_loss, entropy_loss, grad_norm``.

Differences by design: micro-batches are built directly as packed rows (no
pad → unpad round trip), log-probs and entropy come from the fused LM-head
kernel so ``[T, V]`` logits are never materialised, and the loss with all its
statistics is one fused op.
"""
from typing import Dict, List

import torch
import torch.distributed as dist

from chatlearn_b200 import ops
from chatlearn_b200.models.fsdp_module import FSDPModule
from chatlearn_b200.models.nn import FwdCtx
from chatlearn_b200.utils import xfer
from .trainer_utils import pack_samples, split_microbatch, unpack_per_sample


class PolicyTrainer(FSDPModule):
    def setup(self):
        super().setup()
        self._metric_prefix = "policy_trainer" if self.trainable else self.name

    # ------------------------------------------------------------------ helpers
    def _max_reduce(self, n: int) -> int:
        g = self.role_group
        if g is None or g.size == 1:
            return n
        t = torch.tensor([n], dtype=torch.int64, device=self.device)
        g.all_reduce_(t, op=dist.ReduceOp.MAX)
        return int(t.item())

    def _microbatches(self, data_list: List[Dict], for_train: bool):
        ma = self.module_args
        if ma.packing:
            return split_microbatch(data_list, packing=True, max_train_token=ma.max_token_in_packing,
                                    max_reduce=self._max_reduce)
        mbs = ma.train_micro_batch_size if for_train and hasattr(ma, "train_micro_batch_size") \
            else ma.generation_batch_size
        return split_microbatch(data_list, micro_batch_size=max(int(mbs), 1))

    def _num_checkpointed_layers(self, num_tokens: int) -> int:
        """How many leading layers recompute their activations in backward.

        ``checkpoint_layers``: ``all`` (default), an integer, or ``auto``: keep the
        activations of as many layers as fit into the device memory that is free right
        now (autograd saves 4·H + 2·(q+kv) + q + 3·F values per token and dense layer),
        leaving a reserve for the logits chunks, the optimizer step and fragmentation."""
        a = self.model.arch
        L = a.num_hidden_layers
        mode = getattr(self.module_args, "checkpoint_layers", "all")
        if isinstance(mode, int) or str(mode).isdigit():
            return max(0, min(L, int(mode)))
        if str(mode) != "auto" or self.device.type != "cuda":
            return L
        q, kv = a.num_attention_heads * a.head_dim, 2 * a.num_key_value_heads * a.head_dim
        F = a.intermediate_size
        if a.num_experts:
            F = a.moe_intermediate_size * (a.num_experts_per_tok + a.n_shared_experts)
        per_layer = 1.15 * (4 * a.hidden_size + 2 * (q + kv) + q + 3 * F) * 2 * num_tokens
        if self.sp is not None:
            per_layer /= self.sp.size
        free, total = torch.cuda.mem_get_info(self.device)
        free += torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
        keep = int(max(free - 0.10 * total - (6 << 30), 0) // per_layer)
        return max(0, L - keep)

    def _ctx_and_inputs(self, batch):
        """Device tensors + forward context of a packed row (Ulysses-split if sp>1)."""
        batch.to(self.device)
        tokens, positions = batch.tokens, batch.positions
        ctx = FwdCtx(positions=positions, cu_seqlens=batch.cu_seqlens, max_seqlen=batch.max_seqlen,
                     fuse_add_norm=not torch.is_grad_enabled())
        labels = batch.labels
        ctx.row_valid = batch.valid
        if self.sp is not None:
            ctx.sp = self.sp
            ctx.attn_positions = positions
            ctx.row_valid = self.sp.split(batch.valid) if batch.valid is not None else None
            tokens = self.sp.split(tokens)
            labels = self.sp.split(labels)
            ctx.positions = self.sp.split(positions)
        return tokens, labels, ctx

    def _multimodal_embed(self, batch, ctx):
        """Vision-language models: the function that turns this rank's tokens into input embeddings with the tower's
        output in the image rows (and leaves the three-component positions and deep-stack rows in ``ctx``); ``None``
        for text models.  Image rows and positions are addressed in the whole packed row: under Ulysses this rank
        keeps its rows of the embeddings, and the positions stay whole for the attention after the exchange."""
        if getattr(self, "vision", None) is None:
            return None
        from chatlearn_b200.models.nn.vision import multimodal_inputs

        def fn(tokens):
            x = multimodal_inputs(self.model, self.vision, batch.tokens, batch.seq_lens, batch.mm or [], ctx)
            if self.sp is not None:
                n = tokens.shape[0]
                x = self.sp.split(x)
                if ctx.deepstack is not None:
                    rows, taps = ctx.deepstack
                    mine = rows - self.sp.rank * n
                    keep = ((mine >= 0) & (mine < n)).nonzero(as_tuple=True)[0]
                    ctx.deepstack = (mine[keep], [t.index_select(0, keep) for t in taps])
            return x
        return fn

    def _logprobs(self, batch, need_entropy: bool):
        tokens, labels, ctx = self._ctx_and_inputs(batch)
        ctx.aux_weight = getattr(self, "_aux_scale", None)
        if self.resharded:
            # parameter-sharded mode: every block is gathered only while its segment runs, and a segment's
            # activations are recomputed in its backward (which is also where its parameters are re-gathered)
            lp, ent = self.state.logprobs(tokens, labels, ctx, embed_fn=self._multimodal_embed(batch, ctx))
            if self.sp is not None:
                lp, ent = self.sp.gather(lp), self.sp.gather(ent)
            return lp, (ent if need_entropy else None), ctx
        hook = None
        if torch.is_grad_enabled() and getattr(self.module_args, "gradient_checkpointing", False):
            # keep only each layer's input; its activations are recomputed in backward
            from torch.utils.checkpoint import checkpoint
            from chatlearn_b200.models.nn.model import decoder_layer
            arch = self.model.arch

            n_ckpt = self._num_checkpointed_layers(int(tokens.shape[0]))

            def hook(l, p, x, c):
                if l >= n_ckpt:       # the last layers keep their activations: backward reaches them first
                    return decoder_layer(arch, p, x, c, l)
                return checkpoint(lambda xx: decoder_layer(arch, p, xx, c, l), x, use_reentrant=False)
        embed_fn = self._multimodal_embed(batch, ctx)
        x = embed_fn(tokens) if embed_fn is not None else None
        lp, ent = self.model.logprobs(tokens, labels, ctx, layer_hook=hook, x=x)
        if self.sp is not None:
            lp = self.sp.gather(lp)
            ent = self.sp.gather(ent) if need_entropy else None
        return lp, (ent if need_entropy else None), ctx

    # ------------------------------------------------------------------ scoring
    @torch.no_grad()
    def forward_step(self, data_list: List[Dict], iteration: int = 0, **kwargs) -> List[Dict]:
        tag = "old_logprobs" if self.trainable else "ref_logprobs"
        if not data_list:
            return data_list
        pad = self.sp.size if self.sp is not None else 1
        diff_sum, diff_max, diff_n = 0.0, 0.0, 0
        for mb in self._microbatches(data_list, for_train=False):
            if not mb:
                continue
            batch = pack_samples(mb, pad_multiple=pad)
            lp, _, _ = self._logprobs(batch, need_entropy=False)
            for s, v in zip(mb, unpack_per_sample(lp, batch, mb)):
                s[tag] = v
                r = s.get("rollout_logprobs")
                if self.trainable and r is not None and len(r):
                    # how far the engine that generated the tokens and the trainer disagree about their
                    # log-probabilities (same weights: the difference is numerics; a large value means the
                    # rollout ran on other weights or sampled from another distribution than the trainer scores)
                    P, R = int(s["prompt_token_length"]), int(s["response_token_length"])
                    n = min(R, len(r))
                    d = (v[P - 1:P - 1 + n] - torch.as_tensor(r[:n], dtype=torch.float32)).abs()
                    diff_sum += float(d.sum()); diff_max = max(diff_max, float(d.max())); diff_n += n
        if diff_n:
            self._metric_list.append({"rollout_logprob_abs_diff": diff_sum / diff_n, "rollout_logprob_abs_diff_max": diff_max})
        return data_list

    # ------------------------------------------------------------------ training
    def train_step(self, data_list: List[Dict], **kwargs):
        ma = self.module_args
        st = self.state
        # global number of response tokens of this optimizer step (all DP ranks)
        n_local = float(sum(int(s["response_token_length"]) for s in data_list))
        n_tok = torch.tensor([n_local], dtype=torch.float32, device=self.device)
        if self.role_group is not None and self.role_group.size > 1:
            self.role_group.all_reduce_(n_tok)
            if self.sp is not None:
                n_tok /= self.sp.size
        n_global = float(n_tok.item())
        if n_global <= 0.0:
            # nothing to learn from on any rank (all ranks agree: the count was summed over the group):
            # no optimizer step, so AdamW's step count and weight decay do not advance on a zero gradient
            self._logger.warning("train_step: empty mini-batch on every rank, optimizer step skipped")
            return
        inv_norm = 1.0 / max(n_global, 1.0)
        st.zero_grad()
        stats = torch.zeros(6, dtype=torch.float32, device=self.device)
        pad = self.sp.size if self.sp is not None else 1
        need_ent = ma.entropy_coef != 0.0
        use_ref = ma.kl_coef != 0.0
        for mb in self._microbatches(data_list, for_train=True):
            if not mb:
                # ranks with fewer bins still join the collectives of the others
                if self.resharded:
                    st.join_empty_microbatch()
                continue
            batch = pack_samples(mb, pad_multiple=pad)
            self._aux_scale = float(batch.loss_mask.sum()) * inv_norm      # weight of the router losses (below)
            lp, ent, ctx = self._logprobs(batch, need_entropy=True)
            if ma.use_group_sequence_policy:
                loss, s = ops.gspo_loss_fused(
                    lp, batch.old_logprobs, batch.ref_logprobs if use_ref else None, batch.advantages,
                    batch.loss_mask, batch.seq_ids, len(batch.seq_lens), ent if need_ent else ent.detach(),
                    ma.pos_clip_ratio, ma.neg_clip_ratio, ma.diff_clip_ratio, ma.final_clip_ratio,
                    ma.kl_coef, ma.entropy_coef if need_ent else 0.0, inv_norm)
            else:
                loss, s = ops.grpo_loss_fused(
                    lp, batch.old_logprobs, batch.ref_logprobs if use_ref else None,
                    batch.advantages, batch.loss_mask, ent if need_ent else ent.detach(),
                    ma.pos_clip_ratio, ma.neg_clip_ratio, ma.diff_clip_ratio, ma.final_clip_ratio,
                    ma.kl_coef, ma.entropy_coef if need_ent else 0.0, inv_norm)
            for aux in ctx.aux_losses:
                loss = loss + aux * (batch.loss_mask.sum() * inv_norm)
            if self.device.type == "cuda":
                self._logger.debug(f"micro-batch of {batch.num_tokens} tokens: "
                                   f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB allocated before backward")
            loss.backward()
            stats += s.detach()
        grad_norm = st.step()
        # metrics: token means over the whole optimizer step (all ranks)
        if self.role_group is not None and self.role_group.size > 1:
            self.role_group.all_reduce_(stats)
            if self.sp is not None:
                stats /= self.sp.size
        # one device->host read per optimizer step: the loss statistics and the grad norm
        host = xfer.tolist(torch.cat([stats, grad_norm.reshape(1).float()]))
        n = max(host[5], 1.0)
        self._metric_list.append({
            "pg_loss": host[0] / n, "kl_loss": host[1] / n, "entropy_loss": host[2] / n,
            "grad_norm": host[6], "clip_pos_frac": host[3] / n, "clip_neg_frac": host[4] / n,
            "train_tokens": n})
        self._train_iteration += 1
