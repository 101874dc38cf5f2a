"""Policy rollout role backed by the framework's own generation engine.

Parity: chatlearn/models/vllm_module.py:96-598 and
chatlearn/models/sglang_module.py:218-941 (engine set-up, sampling parameters for
train/eval, ``generate``, tagged sleep/wake-up, weight update hooks, output
schema).  There is no external engine: weights live in a TP/EP-sharded
``CausalLM`` in rollout layout and are refreshed by the parameter synchronizer.
"""
import time
from typing import Dict, List, Optional

import torch

from chatlearn_b200.models.base_module import TorchModule
from chatlearn_b200.models.nn import CausalLM, resolve_arch
from chatlearn_b200.parallel import ExpertParallel, build_mesh
from chatlearn_b200.rollout import RolloutEngine, SamplingParams
from chatlearn_b200.synchronizer.parameter_sync import layout_of_model
from chatlearn_b200.utils.constant import TAG_KV_CACHE, TAG_WEIGHTS


class RolloutModule(TorchModule):
    def __init__(self, name: str, args=None, replica_id: int = 0):
        super().__init__(name, args, replica_id)
        self.model: Optional[CausalLM] = None
        self.engine: Optional[RolloutEngine] = None
        self.tp_group = self.ep_group = None
        self.tokenizer = None
        self._metric_prefix = "rollout"

    def init(self):
        ma = self.module_args
        tp = int(ma.tensor_model_parallel_size)
        ep = int(ma.expert_model_parallel_size)
        # a replica spans tp*ep ranks: tp inside, ep across (attention is data parallel over ep)
        self.mesh = build_mesh(self.placement, tp=tp, ep=ep, kinds=("tp", "ep", "dp"))
        self._tp, self._ep = tp, ep
        if self.is_member:
            self.tp_group = self.mesh.groups["tp"]
            self.ep_group = self.mesh.groups["ep"]
            self.role_group = None

    # each EP rank decodes its own sequences, so it is a data-parallel rank of its own
    @property
    def data_parallel_size(self) -> int:
        return self.num_replica * self._ep_size()

    def _ep_size(self):
        return int(getattr(self.module_args, "expert_model_parallel_size", 1) or 1)

    @property
    def data_parallel_rank(self) -> int:
        if self.role_rank < 0:
            return -1
        tp = int(self.module_args.tensor_model_parallel_size)
        return self.role_rank // tp

    @property
    def is_replica_leader(self) -> bool:
        if self.role_rank < 0:
            return False
        return self.role_rank % int(self.module_args.tensor_model_parallel_size) == 0

    @property
    def replica_index(self) -> int:
        return self.data_parallel_rank if self.role_rank >= 0 else 0

    @property
    def num_replica(self) -> int:
        return self._num_replica

    @property
    def loader_parallel_size(self) -> int:
        # every expert-parallel rank of a replica reads its own part of the prompt stream
        return self.data_parallel_size

    @property
    def compute_dtype(self):
        return torch.bfloat16 if self.device.type == "cuda" else torch.float32

    def setup(self):
        if not self.is_member:
            return
        ma = self.module_args
        self.arch = resolve_arch(ma)
        c = self.mesh.coords
        self.model = CausalLM(self.arch, dtype=self.compute_dtype, device=self.device,
                              tp=self._tp, tp_rank=c.get("tp", 0), ep=self._ep, ep_rank=c.get("ep", 0))
        load = getattr(ma, "load", None)
        from chatlearn_b200.checkpoint.safetensors_io import has_safetensors, load_into_model
        if load and has_safetensors(load):
            load_into_model(self.model, load)
        else:
            # placeholder weights; the first parameter sync overwrites them
            self.model.init_weights(int(getattr(ma, "seed", 1234)))
        ep = ExpertParallel(self.ep_group) if self._ep > 1 else None
        self.engine = RolloutEngine(
            self.model, tp_group=self.tp_group if self._tp > 1 else None, ep_group=ep,
            block_size=int(getattr(ma, "kv_block_size", 64)),
            num_blocks=getattr(ma, "num_kv_blocks", None),
            max_num_seqs=int(getattr(ma, "max_num_seqs", 256)),
            max_num_batched_tokens=int(ma.max_num_batched_tokens),
            gpu_memory_utilization=float(ma.gpu_memory_utilization),
            max_model_len=int(ma.seq_length), seed=int(ma.seed) + 7919 * self.replica_index,
            lockstep_group=self.ep_group if self._ep > 1 else None,
            use_cuda_graphs=not bool(getattr(ma, "enforce_eager", False)),
            vision=self._build_vision(load))
        from chatlearn_b200.data.tokenizer import load_tokenizer
        self.tokenizer = load_tokenizer(load, self.arch.vocab_size, kind=str(getattr(ma, "tokenizer", "auto")))

    def _build_vision(self, load):
        from chatlearn_b200.models.nn.vision import attach_vision_block, build_vision_tower
        tower = build_vision_tower(self.arch, self.compute_dtype, self.device, load)
        trainer = getattr(self.global_args.models, "policy_trainer", None)
        if tower is not None and trainer is not None and bool(getattr(trainer, "train_vision_tower", False)):
            # the trainer updates the tower: its weights join this model's blocks and arrive with every weight sync
            attach_vision_block(self.model, tower)
        return tower

    # ------------------------------------------------------------------ generation
    def _sampling_params(self, is_eval: bool, max_tokens: int) -> SamplingParams:
        ma = self.module_args
        p = "eval_" if is_eval else ""
        return SamplingParams(
            temperature=getattr(ma, p + "temperature"), top_p=getattr(ma, p + "top_p"),
            top_k=getattr(ma, p + "top_k"), min_p=getattr(ma, "min_p", 0.0),
            presence_penalty=getattr(ma, p + "presence_penalty"),
            frequency_penalty=getattr(ma, p + "frequency_penalty"),
            repetition_penalty=getattr(ma, p + "repetition_penalty"), max_tokens=max_tokens,
            ignore_eos=bool(getattr(ma, "ignore_eos", False)))

    def generate(self, data_list: List[Dict], is_eval: bool = False):
        ma = self.module_args
        key = ma.vllm_input_ids_key
        prompts, budgets = [], []
        for s in data_list:
            ids = list(s[key])
            prompts.append(ids)
            # per-sample budget (partial rollout sets max_generate_token_length)
            b = int(s.get("max_generate_token_length", ma.max_response_tokens_length))
            budgets.append(min(b, ma.seq_length - len(ids)))
        sp = self._sampling_params(is_eval, ma.max_response_tokens_length)
        mm = None
        if self.engine.vision is not None:
            mm = [{"pixel_values": s["pixel_values"], "image_grid_thw": s["image_grid_thw"],
                   "visual_time_steps": s.get("visual_time_steps")}
                  if s.get("pixel_values") is not None else None for s in data_list]
        return self.engine.generate(prompts, sp, max_new_tokens=budgets, mm_inputs=mm)

    def postprocess_func(self, data_list: List[Dict], seqs) -> List[Dict]:
        out = []
        for s, q in zip(data_list, seqs):
            r = dict(s)
            prompt_ids = list(s.get("prompt_token_ids", s[self.module_args.vllm_input_ids_key]))
            full_in = list(s[self.module_args.vllm_input_ids_key])
            resp = full_in[len(prompt_ids):] + q.output          # earlier partial rounds + this round
            r["all_tokens"] = torch.tensor(prompt_ids + resp, dtype=torch.long)
            r["prompt_token_length"] = len(prompt_ids)
            r["response_token_length"] = len(resp)
            r["all_token_length"] = len(prompt_ids) + len(resp)
            r["str_outputs"] = self.tokenizer.decode(resp, skip_special_tokens=True) \
                if self.tokenizer is not None else ""
            r["finish_reason"] = q.finish_reason
            r["rollout_logprobs"] = torch.tensor(q.logprobs, dtype=torch.float32)
            if "rollout_round" in r:
                r["rollout_round"] += 1
            out.append(r)
        return out

    def forward_step(self, data_list: List[Dict], iteration: int = 0, is_eval: bool = False, **kw):
        cached = self.load_stage_outputs(is_eval, iteration)
        if cached is not None:
            return cached
        t0 = time.perf_counter()
        seqs = self.generate(data_list, is_eval)
        out = self.postprocess_func(data_list, seqs)
        dt = time.perf_counter() - t0
        if not is_eval and out:
            lens = torch.tensor([o["response_token_length"] for o in out], dtype=torch.float32)
            mx = self.module_args.max_response_tokens_length
            self._metric_list.append({
                "response_length": lens.mean().item(), "response_length_max": lens.max().item(),
                "response_clip_ratio": (lens >= mx).float().mean().item(),
                "prompt_length": sum(o["prompt_token_length"] for o in out) / len(out),
                "response_p25": lens.quantile(0.25).item(), "response_p50": lens.quantile(0.5).item(),
                "response_p75": lens.quantile(0.75).item(),
                "gen_tokens_per_s": lens.sum().item() / max(dt, 1e-9),
                "preemptions": float(self.engine.stats.get("preemptions", 0)),
                **{k: float(self.engine.stats.get(k, 0)) for k in
                   ("prefill_s", "decode_s", "sched_s", "prefill_steps", "decode_steps")}})
        self.save_stage_outputs(is_eval, out, iteration)
        return out

    def eval_forward(self, data_list, iteration: int = 0, **kw):
        return self.forward_step(data_list, iteration, is_eval=True)

    # ------------------------------------------------------------------ memory tags
    def offload(self, tags=None, **kwargs):
        if not self.is_member or self.engine is None:
            return
        fg = self.module_args.free_gpu_memory
        tags = tags or ([TAG_KV_CACHE] + ([TAG_WEIGHTS] if fg.offload_weights else []))
        if TAG_KV_CACHE in tags:
            self.engine.free_kv_cache()
        if TAG_WEIGHTS in tags and self._resident["weights"]:
            # rollout weights are a derived copy: drop them, the next sync rebuilds them
            for b in self.model.blocks:
                self._release(b, "flat")
            self._resident["weights"] = False
        self.empty_cache()
        if self.device.type == "cuda":
            self._logger.debug(f"offload({tags}) -> {torch.cuda.memory_allocated() / 2**30:.1f} GiB allocated")

    def onload(self, tags=None, **kwargs):
        if not self.is_member or self.engine is None:
            return
        tags = tags or [TAG_WEIGHTS, TAG_KV_CACHE]
        if TAG_WEIGHTS in tags and not self._resident["weights"]:
            for b in self.model.blocks:
                b.bind(torch.empty(b.numel, dtype=b.dtype, device=self.device))
            self._resident["weights"] = True
            self.engine.invalidate_graphs()
        if TAG_KV_CACHE in tags:
            self.engine.alloc_kv_cache()

    def _release(self, owner, attr):
        owner.flat = None
        for p in owner.params.values():
            p.data = torch.empty(0, dtype=owner.dtype, device=owner.device)

    # ------------------------------------------------------------------ parameter sync (destination)
    def sync_layout(self):
        return layout_of_model(self.model, self.get_rank(), prefix=f"{self.name}/")

    def sync_buffers(self) -> Dict[str, torch.Tensor]:
        return {f"{self.name}/{b.name}": b.flat for b in self.model.blocks}

    def dump_parameters(self, path: str):
        import os
        os.makedirs(path, exist_ok=True)
        import dataclasses
        m = self.model
        torch.save({"leaves": {n: p.detach().float().cpu() for n, p, _, _ in m.named_leaves()},
                    "arch": dataclasses.asdict(m.arch), "tp": m.tp, "tp_rank": m.tp_rank, "ep": m.ep,
                    "ep_rank": m.ep_rank},
                   os.path.join(path, f"{self.name}_rank{self.get_rank()}.pt"))
