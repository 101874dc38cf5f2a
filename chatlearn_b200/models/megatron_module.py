"""Megatron-style worker: tensor / pipeline / context / expert parallel model role.

Parity: chatlearn/models/megatron_module.py:65-331 (distributed initialisation,
memory managers, checkpoint hooks, global parameter naming for PP/VPP layer
offsets and EP expert offsets, parameter metadata for the synchronizer).  The
reference delegates the model and its parallel runtime to Megatron-Core; here the
role builds this framework's ``CausalLM`` with TP/EP-sharded leaves for its
pipeline stage, wires the process groups of ``parallel.mesh`` into the forward
context, and shards the optimizer state over the (data x context) parallel group
(dense leaves) and the expert-data-parallel group (expert leaves), i.e. the
distributed optimizer.  Global naming is implicit: every leaf carries the HF
tensor rectangles it holds, so PP layer offsets and EP expert offsets need no
separate translation step.
"""
import math
import os
from typing import List, Optional, Tuple


from chatlearn_b200 import ops

from chatlearn_b200.models.fsdp_module import FSDPModule
from chatlearn_b200.models.nn import CausalLM, ModelArch, resolve_arch
from chatlearn_b200.parallel import ContextParallel, ExpertParallel, build_mesh
from chatlearn_b200.parallel.zero import ShardedTrainState
from chatlearn_b200.synchronizer.parameter_sync import layout_of_model


def arch_from_megatron_cfg(mc) -> ModelArch:
    """``MegatronModelArchitectureConfig`` → ``ModelArch`` (inverse of
    ``utils.megatron_utils.update_cfg``)."""
    moe = mc.num_experts is not None and mc.num_experts > 0
    mla = bool(mc.multi_latent_attention)
    return ModelArch(
        model_type="deepseek_v3" if mla else ("qwen3_moe" if moe else ("qwen3" if mc.qk_layernorm else "llama")),
        vocab_size=mc.vocab_size, hidden_size=mc.hidden_size, num_hidden_layers=mc.num_layers,
        num_attention_heads=mc.num_attention_heads,
        num_key_value_heads=mc.num_query_groups or mc.num_attention_heads,
        head_dim=(mc.qk_head_dim + mc.qk_pos_emb_head_dim) if mla else mc.kv_channels,
        intermediate_size=mc.ffn_hidden_size, rms_norm_eps=mc.norm_epsilon, rope_theta=float(mc.rotary_base),
        max_position_embeddings=mc.max_position_embeddings, qk_norm=mc.qk_layernorm,
        attention_bias=mc.add_qkv_bias, tie_word_embeddings=not mc.untie_embeddings_and_output_weights,
        num_experts=mc.num_experts or 0, num_experts_per_tok=mc.moe_router_topk if moe else 0,
        moe_intermediate_size=mc.moe_ffn_hidden_size or 0, router_aux_loss_coef=mc.moe_aux_loss_coeff,
        n_shared_experts=((mc.moe_shared_expert_intermediate_size or 0) // max(mc.moe_ffn_hidden_size or 1, 1)),
        first_k_dense_replace=(mc.moe_layer_freq.index(1) if isinstance(mc.moe_layer_freq, list)
                               and 1 in mc.moe_layer_freq else 0),
        scoring_func=mc.moe_router_score_function, n_group=mc.moe_router_num_groups or 1,
        topk_group=mc.moe_router_group_topk or 1, routed_scaling_factor=mc.moe_router_topk_scaling_factor or 1.0,
        router_bias=mc.moe_router_enable_expert_bias, kv_lora_rank=mc.kv_lora_rank if mla else 0,
        q_lora_rank=mc.q_lora_rank, qk_nope_head_dim=mc.qk_head_dim if mla else 0,
        qk_rope_head_dim=mc.qk_pos_emb_head_dim if mla else 0, v_head_dim=(mc.v_head_dim or 0) if mla else 0)


def pipeline_stage_sizes(num_layers: int, pp: int, first: Optional[int] = None, last: Optional[int] = None) -> List[int]:
    """Layers per pipeline stage; ``first`` / ``last`` fix the size of the first and last stage (uneven
    pipelines, megatron_config ``decoder_first/last_pipeline_num_layers``), the others share the rest."""
    if pp == 1:
        return [num_layers]
    sizes = [0] * pp
    rem, mids = num_layers, list(range(pp))
    if first is not None:
        sizes[0] = first
        rem -= first
        mids.remove(0)
    if last is not None:
        sizes[-1] = last
        rem -= last
        mids.remove(pp - 1)
    base, extra = divmod(rem, len(mids)) if mids else (0, 0)
    assert mids or rem == 0, "the first and last stage must hold all layers of a two-stage pipeline"
    for i, st in enumerate(mids):
        sizes[st] = base + (1 if i < extra else 0)
    return sizes


def pipeline_layer_range(num_layers: int, pp: int, stage: int, first: Optional[int] = None,
                         last: Optional[int] = None) -> Tuple[int, int]:
    """Layers of a pipeline stage."""
    sizes = pipeline_stage_sizes(num_layers, pp, first, last)
    lo = sum(sizes[:stage])
    return lo, lo + sizes[stage]


def pipeline_chunk_ranges(num_layers: int, pp: int, vpp: int, stage: int, first: Optional[int] = None,
                          last: Optional[int] = None) -> List[Tuple[int, int]]:
    """Layer ranges of the ``vpp`` model chunks a stage holds under the interleaved schedule: every stage cuts its
    layers into ``vpp`` equal chunks, and the model runs through chunk 0 of all stages, then chunk 1 of all stages and
    so on, so chunk ``c`` of the model lives on stage ``c % pp`` (Megatron's
    ``virtual_pipeline_model_parallel_size``; chatlearn/configs/megatron_config.py:106 passes it through, and
    chatlearn/models/megatron_module.py:259-283 names the layers by the same offsets).  With ``first`` / ``last`` the
    chunks of the first and last stage have their own size."""
    sizes = pipeline_stage_sizes(num_layers, pp, first, last)
    assert all(n % vpp == 0 for n in sizes), \
        f"stages of {sizes} layers do not split into {vpp} chunks of equal size"
    per = [n // vpp for n in sizes]
    round_layers = sum(per)
    lo = sum(per[:stage])
    return [(j * round_layers + lo, j * round_layers + lo + per[stage]) for j in range(vpp)]


class MegatronModule(FSDPModule):
    """Shares checkpoint / residency plumbing with the FSDP-style role; differs in
    how the model is partitioned and which groups reduce what."""

    def init(self):
        ma = self.module_args
        self.tp_size = int(ma.tensor_model_parallel_size)
        self.pp_size = int(ma.pipeline_model_parallel_size)
        self.cp_size = int(ma.context_parallel_size)
        self.ep_size = int(ma.expert_model_parallel_size)
        self.etp_size = int(ma.expert_tensor_parallel_size or 1)
        self.vpp_size = int(getattr(ma, "virtual_pipeline_model_parallel_size", None) or 1)
        assert self.vpp_size == 1 or self.pp_size > 1, "model chunks (virtual pipeline) need pipeline parallelism"
        assert self.etp_size in (1, self.tp_size), \
            "expert tensor parallelism is either off or spans the tensor-parallel group (etp == tp)"
        self.mesh = build_mesh(self.placement, tp=self.tp_size, cp=self.cp_size, pp=self.pp_size,
                               ep=self.ep_size, etp=self.etp_size,
                               kinds=("tp", "cp", "dp", "pp", "ep", "edp", "dp_cp", "mp"))
        self.sp = None
        # Megatron's sequence parallelism: between the tensor-parallel layers every rank keeps 1/tp of the rows
        self.seq_parallel = self.tp_size > 1 and bool(getattr(ma, "sequence_parallel", False))
        if self.is_member:
            g = self.mesh.groups
            self.tp_group, self.cp_group, self.pp_group = g["tp"], g["cp"], g["pp"]
            self.ep_group, self.edp_group = g["ep"], g["edp"]
            self.dp_group = g["dp_cp"]            # gradients of dense leaves reduce over dp x cp
            self.role_group = g["dp_cp"]
            self.mp_group = g["mp"]               # ranks that share one data shard (tp x cp x pp)
            c = self.mesh.coords
            self.pp_rank, self.tp_rank, self.cp_rank, self.ep_rank = c["pp"], c["tp"], c["cp"], c["ep"]

    @property
    def is_data_leader(self) -> bool:
        if not self.is_member:
            return False
        c = self.mesh.coords
        return c["tp"] == 0 and c["cp"] == 0 and c["pp"] == self.pp_size - 1

    @property
    def data_parallel_size(self) -> int:
        return max(len(self.placement) // (self.tp_size * self.cp_size * self.pp_size), 1)

    @property
    def data_parallel_rank(self) -> int:
        return self.mesh.coords.get("dp", 0) if self.is_member else -1

    @property
    def is_first_stage(self):
        return self.pp_rank == 0

    @property
    def is_last_stage(self):
        return self.pp_rank == self.pp_size - 1

    def resolve_arch(self) -> ModelArch:
        ma = self.module_args
        if getattr(ma, "model_arch", None) or (ma.load and os.path.exists(os.path.join(ma.load, "config.json"))):
            return resolve_arch(ma)
        return arch_from_megatron_cfg(ma.megatron_model_cfg)

    def create_model(self) -> CausalLM:
        ma = self.module_args
        arch = self.resolve_arch()
        if self.vpp_size > 1:
            ranges = pipeline_chunk_ranges(arch.num_hidden_layers, self.pp_size, self.vpp_size, self.pp_rank,
                                           ma.decoder_first_pipeline_num_layers, ma.decoder_last_pipeline_num_layers)
        else:
            ranges = pipeline_layer_range(arch.num_hidden_layers, self.pp_size, self.pp_rank,
                                          ma.decoder_first_pipeline_num_layers, ma.decoder_last_pipeline_num_layers)
        pad = math.lcm(self.dp_group.size, self.edp_group.size)
        model = CausalLM(arch, dtype=self.compute_dtype, device=self.device, tp=self.tp_size, tp_rank=self.tp_rank,
                         ep=self.ep_size, ep_rank=self.ep_rank, etp=self.etp_size,
                         etp_rank=self.tp_rank if self.etp_size > 1 else 0, layer_range=ranges,
                         with_embed=self.is_first_stage or (arch.tie_word_embeddings and self.is_last_stage),
                         with_head=self.is_last_stage, pad_to=pad)
        from chatlearn_b200.checkpoint.safetensors_io import has_safetensors, load_into_model
        if ma.load and has_safetensors(ma.load):
            load_into_model(model, ma.load)
        else:
            model.init_weights(int(ma.seed))
        return model

    def setup(self):
        if not self.is_member:
            return
        self.arch = self.resolve_arch()
        self.model = self.create_model()
        self.ep = ExpertParallel(self.ep_group) if self.ep_size > 1 else None
        # vision-language models: every stage needs the (time, row, column) positions, the first stage also the
        # tower's embeddings (and, when the tower is trained, its weights as one more parameter block)
        from chatlearn_b200.models.nn.vision import attach_vision_block, build_vision_tower
        self.vision = build_vision_tower(self.arch, self.compute_dtype, self.device, getattr(self.module_args, "load", None))
        if self.vision is not None:
            if self.trainable and self.is_first_stage and bool(getattr(self.module_args, "train_vision_tower", False)):
                attach_vision_block(self.model, self.vision, pad_to=math.lcm(self.dp_group.size, self.edp_group.size))
        if self.seq_parallel:
            # norms and routers see only this rank's rows: their gradients are partial sums over the group
            for b in self.model.blocks:
                for lf in b.leaves:
                    if b.short(lf.name) in ("input_layernorm", "post_attention_layernorm", "norm", "router",
                                            "shared_expert_gate"):
                        lf.grad_sum_tp = True
                    # experts kept whole on every tensor-parallel rank work on that rank's rows only
                    if b.short(lf.name) in ("w13", "w2") and self.etp_size == 1 and self.ep_size == 1:
                        lf.grad_sum_tp = True
        if self.seq_parallel and self.device.type == "cuda" and self.trainable and ops.get_mode() == "native":
            # row-parallel layers: product and reduce-scatter in one pass over peer memory
            from chatlearn_b200.parallel import symm_collectives
            symm_collectives.attach_gemm_reduce_scatter(self.tp_group)
            # and the gathers of the sequence-parallel rows in front of the column-parallel layers as peer stores
            symm_collectives.attach_exchange(self.tp_group)
        self.cp = ContextParallel(self.cp_group) if self.cp_size > 1 else None
        if self.cp is not None:
            from chatlearn_b200.parallel import symm_collectives
            symm_collectives.attach_exchange(self.cp_group)
        if self.trainable:
            oc = self.module_args.optimizer
            extra = [g for g in (self.tp_group, self.pp_group) if g.size > 1]
            self.state = ShardedTrainState(
                self.model, self.dp_group, self.edp_group if self.ep_size > 1 else None, lr=oc.lr,
                betas=(oc.adam_beta1, oc.adam_beta2), eps=getattr(oc, "adam_eps", 1e-8),
                weight_decay=oc.weight_decay, clip_grad=oc.clip_grad, extra_norm_groups=extra,
                tp_size=self.tp_size, ep_group=self.ep_group if self.ep_size > 1 else None,
                tp_group=self.tp_group if self.tp_size > 1 else None)
            if self.pp_size > 1 and self.arch.tie_word_embeddings:
                # the first and the last stage hold copies of the tied embedding: half of its squared norm each
                self.state.block_norm_weight["embed"] = 0.5

    # ------------------------------------------------------------------ checkpoints (Megatron layout)
    def checkpoint_dir(self, iteration: int) -> str:
        return os.path.join(self.runtime_args.output_dir, "save_model", self.name)

    def save_checkpoint(self, iteration: int):
        """``iter_{it:07d}/mp_rank_{tp:02d}[_{pp:03d}][_{ep:03d}]/model_optim_rng.pt`` +
        ``latest_checkpointed_iteration.txt``; one writer per model-parallel rank
        (data-parallel rank 0), optimizer shards per data-parallel rank alongside."""
        if not self.is_member or self.model is None:
            return
        from chatlearn_b200.checkpoint.megatron_ckpt import save_megatron_checkpoint
        save_megatron_checkpoint(self, self.checkpoint_dir(iteration), iteration)
        if self.role_group is not None:
            self.role_group.barrier()

    def load_checkpoint(self, path: str):
        from chatlearn_b200.checkpoint.megatron_ckpt import load_megatron_checkpoint
        return load_megatron_checkpoint(self, path)

    # ------------------------------------------------------------------ sync metadata (API parity)
    def map_local_param_name_to_global(self) -> List[str]:
        """HF tensor names this rank holds a part of (the reference's "global names")."""
        names = []
        for _, _, lf, _ in self.model.named_leaves():
            for s in lf.segments:
                if s.hf_name not in names:
                    names.append(s.hf_name)
        return names

    def get_parameter_metadata(self):
        return layout_of_model(self.model, self.get_rank(), prefix=f"{self.name}/")
