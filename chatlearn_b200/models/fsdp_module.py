"""FSDP-style worker: a replicated-compute / sharded-optimizer model role.

Parity: chatlearn/models/fsdp_module.py:188-660 (device mesh, model creation,
sharding, optimizer, weight export for sync, offload, checkpoints, RNG state).
The reference wraps a HuggingFace model with torch ``fully_shard``; this module
builds the framework's own ``CausalLM`` over flat parameter blocks and shards the
optimizer state with ``parallel.zero.ShardedTrainState``.  ``fsdp_size`` smaller
than the role's GPU count is hybrid sharding (HSDP, the reference's 2-D device mesh
``(replicate, shard)``): neighbouring ranks form shard groups of ``fsdp_size`` that
reduce-scatter gradients and all-gather parameters among themselves, and the ranks
holding the same shard in different groups all-reduce their gradient shards.
"""
import os
import random
from typing import Dict, List, Optional

import numpy as np
import torch

from chatlearn_b200 import ops
from chatlearn_b200.models.base_module import TorchModule
from chatlearn_b200.models.nn import CausalLM, resolve_arch
from chatlearn_b200.parallel import UlyssesGroup, build_mesh
from chatlearn_b200.parallel.zero import ShardedTrainState
from chatlearn_b200.synchronizer.parameter_sync import layout_of_model


class FSDPModule(TorchModule):
    def __init__(self, name: str, args=None, replica_id: int = 0):
        super().__init__(name, args, replica_id)
        self.model: Optional[CausalLM] = None
        self.state: Optional[ShardedTrainState] = None
        self.sp: Optional[UlyssesGroup] = None
        self.dp_group = self.role_group = None

    # ------------------------------------------------------------------ groups
    def init(self):
        sp = int(getattr(self.module_args, "ulysses_sequence_parallel_size", 1) or 1)
        n = len(self.placement)
        fs = int(getattr(self.module_args, "fsdp_size", n) or n)
        hybrid = 0 < fs < n and n % fs == 0
        kinds = ("dp", "sp", "dp_outer") + (("dp_shard", "dp_rep") if hybrid else ())
        self.mesh = build_mesh(self.placement, sp=sp, kinds=kinds, shard=fs if hybrid else 0)
        self.shard_group = self.replica_group = None
        if self.is_member:
            self.role_group = self.mesh.groups["dp"]
            self.dp_group = self.mesh.groups["dp"]           # gradient reduction: all ranks
            # optimizer-state shards: the whole role, or its shard group under hybrid sharding
            self.shard_group = self.mesh.groups["dp_shard"] if hybrid else self.dp_group
            self.replica_group = self.mesh.groups["dp_rep"] if hybrid else None
            self.dp_outer_group = self.mesh.groups["dp_outer"]
            if sp > 1:
                self.sp = UlyssesGroup(self.mesh.groups["sp"])
                from chatlearn_b200.parallel import symm_collectives
                symm_collectives.attach_exchange(self.mesh.groups["sp"])

    @property
    def is_data_leader(self) -> bool:
        return self.is_member and self.mesh.coords.get("sp", 0) == 0

    @property
    def resharded(self) -> bool:
        return bool(getattr(self.state, "reshard", False))

    @property
    def compute_dtype(self):
        return torch.bfloat16 if self.device.type == "cuda" else torch.float32

    # ------------------------------------------------------------------ model
    def create_model(self) -> CausalLM:
        arch = resolve_arch(self.module_args)
        dp = self.shard_group.size if self.shard_group is not None else 1
        # blocks padded so that every rank's shard is a whole number of 16-byte vectors
        model = CausalLM(arch, dtype=self.compute_dtype, device=self.device, pad_to=dp * 8)
        load = getattr(self.module_args, "load", None)
        from chatlearn_b200.checkpoint.safetensors_io import has_safetensors, load_into_model
        if load and has_safetensors(load):
            load_into_model(model, load)
        else:
            model.init_weights(int(getattr(self.module_args, "seed", 1234)))
        return model

    def setup(self):
        if not self.is_member:
            return
        self.arch = resolve_arch(self.module_args)
        self.model = self.create_model()
        # vision-language roles keep a frozen copy of the vision tower beside the language model
        from chatlearn_b200.models.nn.vision import build_vision_tower
        self.vision = build_vision_tower(self.arch, self.compute_dtype, self.device, getattr(self.module_args, "load", None))
        if self.vision is not None:
            if self.trainable and bool(getattr(self.module_args, "train_vision_tower", False)):
                # the tower's weights become one more parameter block: sharded optimizer state, gradient
                # reduction, offload, checkpoints and the weight sync into the rollout engine cover it
                from chatlearn_b200.models.nn.vision import attach_vision_block
                dp = self.shard_group.size if self.shard_group is not None else 1
                attach_vision_block(self.model, self.vision, pad_to=dp * 8)
        if self.trainable:
            oc = self.module_args.optimizer
            grad_dtype = torch.float32
            gd = str(getattr(self.module_args, "grad_dtype", "fp32"))
            if gd in ("bf16", "param"):
                grad_dtype = self.compute_dtype
            # parameter-sharded mode (FSDP2 ``reshard_after_forward``): 1/dp of parameters, gradients and
            # optimizer state resident; blocks are gathered only while their segment runs
            state_cls = ShardedTrainState
            if bool(getattr(self.module_args, "reshard_after_forward", False)):
                from chatlearn_b200.parallel.fsdp2 import ReshardedTrainState
                state_cls = ReshardedTrainState
            extra = {}
            if self.replica_group is not None:
                extra["replica_group"] = self.replica_group
            self.state = state_cls(
                self.model, self.shard_group, lr=oc.lr, betas=(oc.adam_beta1, oc.adam_beta2),
                eps=getattr(oc, "adam_eps", 1e-8), weight_decay=oc.weight_decay,
                clip_grad=oc.clip_grad, grad_dtype=grad_dtype, **extra)
            # optimizer-step collectives by this package's peer-memory kernels; needs the
            # weights and gradient buffers to stay on the device (symmetric memory)
            fg = self.module_args.free_gpu_memory
            if bool(getattr(self.module_args, "fused_optimizer_comm", True)) and not fg.offload_weights \
                    and not self.resharded \
                    and os.environ.get("CLB200_SYMM_ZERO", "1") != "0" and ops.get_mode() == "native":
                if self.state.enable_symm():
                    self._logger.info("optimizer step uses in-kernel reduce-scatter / all-gather over symmetric memory")
            if self.resume_training_path():
                self.load_checkpoint(self.resume_training_path())

    def resume_training_path(self) -> Optional[str]:
        if not getattr(self, "_resume_training", False):
            return None
        root = os.path.join(self.runtime_args.output_dir, "save_model", self.name)
        if not os.path.isdir(root):
            return None
        its = sorted(int(d) for d in os.listdir(root) if d.isdigit())
        return os.path.join(root, str(its[-1])) if its else None

    # ------------------------------------------------------------------ residency
    def _tagged(self, tag: str):
        if self.state is not None:
            return self.state.tensors_for(tag)
        if tag == "weights" and self.model is not None:
            return [(b, "flat") for b in self.model.blocks]
        return []

    def _release(self, owner, attr):
        if attr == "flat":
            owner.flat = None
            for p in owner.params.values():
                p.data = torch.empty(0, dtype=owner.dtype, device=owner.device)
        elif attr == "grad":
            owner.grad = None
            for p in owner.block.params.values():
                p.grad = None
                if hasattr(p, "main_grad"):
                    p.main_grad = None
        else:
            setattr(owner, attr, None)

    def _rebind(self, owner, attr, tensor):
        if attr == "flat":
            owner.bind(tensor)
        else:
            setattr(owner, attr, tensor)

    def _weights_regenerable(self) -> bool:
        fg = self.module_args.free_gpu_memory
        if self.resharded:
            return False
        return (self.trainable and self.state is not None and self.state.symm is None
                and not fg.offload_optimizer_states and self._resident.get("optimizer", True))

    def _regenerate_weights(self):
        """bf16 weights = cast of the fp32 master shards (all-gathered over the data-parallel group)."""
        for s in self.state.states:
            if s.block.flat is None:
                s.block.bind(torch.empty(s.block.numel, dtype=s.block.dtype, device=self.device))
        self.state.rebuild_params()

    def _build_grad_buffers(self):
        if self.state is None:
            return
        if self.resharded:
            for s in self.state.states:       # only the resident 1/dp accumulator; whole-block buffers are pooled
                if s.grad_shard is None:
                    s.grad_shard = torch.zeros(s.shard_numel, dtype=torch.float32, device=self.device)
            return
        for s in self.state.states:
            if s.grad is None:
                gd = self.compute_dtype if str(getattr(
                    self.module_args, "grad_dtype", "fp32")) in ("bf16", "param") else torch.float32
                s.grad = torch.zeros(s.block.numel, dtype=gd, device=self.device)
                s.block.enable_grad(s.grad)
            if s.grad_shard is None:
                s.grad_shard = s.grad if (s.group.size == 1 and s.grad.dtype == torch.float32) else \
                    torch.zeros(s.shard_numel, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------ parameter sync (source side)
    def sync_layout(self):
        if self.resharded:
            # every rank publishes the slice of each block it holds: the rollout ranks pull what they need from
            # all of them (over NVLink where the slices live in symmetric memory)
            rng = {s.block.name: (s.lo, s.hi) for s in self.state.states}
            return layout_of_model(self.model, self.get_rank(), lambda name: rng[name], prefix=f"{self.name}/")
        return layout_of_model(self.model, self.get_rank(), prefix=f"{self.name}/")

    def sync_buffers(self) -> Dict[str, torch.Tensor]:
        if self.resharded:
            return {f"{self.name}/{s.block.name}": s.param_shard for s in self.state.states}
        return {f"{self.name}/{b.name}": b.flat for b in self.model.blocks}

    def get_fsdp_param_name(self, block_size: int = 3_000_000_000) -> List[List[str]]:
        """HF parameter names grouped into blocks of at most ``block_size`` elements
        (API of chatlearn/models/fsdp_module.py:401-418)."""
        out, cur, n = [], [], 0
        from chatlearn_b200.models.nn.layout import hf_tensor_shapes
        for name, shp in hf_tensor_shapes(self.arch).items():
            m = int(np.prod(shp))
            if cur and n + m > block_size:
                out.append(cur)
                cur, n = [], 0
            cur.append(name)
            n += m
        if cur:
            out.append(cur)
        return out

    # ------------------------------------------------------------------ checkpoints
    def checkpoint_dir(self, iteration: int) -> str:
        return os.path.join(self.runtime_args.output_dir, "save_model", self.name, str(iteration))

    def get_rng_state(self):
        st = {"cpu": torch.get_rng_state(), "numpy": np.random.get_state(), "random": random.getstate()}
        if self.device.type == "cuda":
            st["cuda"] = torch.cuda.get_rng_state(self.device)
        return st

    def set_rng_state(self, st):
        torch.set_rng_state(st["cpu"])
        np.random.set_state(st["numpy"])
        random.setstate(st["random"])
        if "cuda" in st and self.device.type == "cuda":
            torch.cuda.set_rng_state(st["cuda"], self.device)

    def save_checkpoint(self, iteration: int):
        """Per-rank files ``model_world_size_{W}_rank_{R}.pt``, ``optim_…pt``,
        ``extra_state_…pt`` (layout of chatlearn/models/fsdp_module.py:577-621) and,
        when ``save_hf``, a HuggingFace directory written by rank 0."""
        if not self.is_member or self.model is None:
            return
        d = self.checkpoint_dir(iteration)
        os.makedirs(d, exist_ok=True)
        W, R = len(self.placement), self.role_rank
        if self.state is not None:
            model_sd = {s.block.name: {"shard": s.master.cpu(), "lo": s.lo, "hi": s.hi,
                                       "numel": s.block.numel} for s in self.state.states}
            sd = self.state.state_dict()
            optim_sd = {"step": sd["step"], "blocks": {k: {"exp_avg": v["exp_avg"], "exp_avg_sq": v["exp_avg_sq"]}
                                                       for k, v in sd["blocks"].items()}}
            torch.save(optim_sd, os.path.join(d, f"optim_world_size_{W}_rank_{R}.pt"))
        else:
            model_sd = {b.name: {"shard": b.flat.float().cpu(), "lo": 0, "hi": b.numel, "numel": b.numel}
                        for b in self.model.blocks}
        torch.save(model_sd, os.path.join(d, f"model_world_size_{W}_rank_{R}.pt"))
        torch.save({"rng": self.get_rng_state(), "iteration": iteration},
                   os.path.join(d, f"extra_state_world_size_{W}_rank_{R}.pt"))
        if getattr(self.module_args, "save_hf", False):
            from chatlearn_b200.checkpoint.safetensors_io import save_hf_checkpoint
            if self.resharded:
                with self.state.all_gathered() as whole:        # collective: every rank gathers, rank 0 writes
                    if R == 0:
                        save_hf_checkpoint(whole, os.path.join(d, "huggingface"))
            elif R == 0:
                save_hf_checkpoint(self.model, os.path.join(d, "huggingface"))
        if self.role_group is not None:
            self.role_group.barrier()

    def load_checkpoint(self, path: str):
        W, R = len(self.placement), self.role_rank
        mp = os.path.join(path, f"model_world_size_{W}_rank_{R}.pt")
        if not os.path.exists(mp):
            return False
        model_sd = torch.load(mp, weights_only=False)
        if self.state is not None:
            op = os.path.join(path, f"optim_world_size_{W}_rank_{R}.pt")
            optim_sd = torch.load(op, weights_only=False) if os.path.exists(op) else None
            blocks = {}
            for s in self.state.states:
                b = model_sd[s.block.name]
                ob = optim_sd["blocks"][s.block.name] if optim_sd else None
                blocks[s.block.name] = {
                    "master": b["shard"], "lo": b["lo"], "hi": b["hi"], "numel": b["numel"],
                    "exp_avg": ob["exp_avg"] if ob else torch.zeros_like(b["shard"]),
                    "exp_avg_sq": ob["exp_avg_sq"] if ob else torch.zeros_like(b["shard"])}
            self.state.load_state_dict({"step": optim_sd["step"] if optim_sd else 0, "blocks": blocks})
        else:
            for b in self.model.blocks:
                b.flat.copy_(model_sd[b.name]["shard"])
        ep = os.path.join(path, f"extra_state_world_size_{W}_rank_{R}.pt")
        if os.path.exists(ep):
            self.set_rng_state(torch.load(ep, weights_only=False)["rng"])
        return True
