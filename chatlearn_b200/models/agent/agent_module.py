"""Rollout role for agent tasks: many multi-turn trajectories, one engine call per turn.

Parity: chatlearn/models/agent/agent_module.py:27-120 (graph registry,
``generate_per_request``, ``postprocess_func`` field names).  The reference runs one
coroutine per request against an async SGLang server.  Here every trajectory is a
generator (see ``chat_model``) and the engine is driven through an open session
(``rollout/engine.py::RolloutSession``): each model turn is submitted as its own
request, the engine steps, and a trajectory whose request finished in that step runs
its tools and submits its next turn before the next step: it joins the running batch
without waiting for the other trajectories' turns (``agent_scheduling: continuous``,
the default).  ``agent_scheduling: lockstep`` answers all waiting requests with one
batched call per round instead.  Tools run on the replica's first tensor-parallel
rank; the requests it submits are broadcast so that all ranks of the replica feed
their engines the same way.
"""
from typing import Dict, List, Type

import torch

from chatlearn_b200.models.rollout_module import RolloutModule
from chatlearn_b200.rollout.engine import SamplingParams
from .base_agent_graph import AgentGraphOutput, BaseAgentGraph
from .chat_model import LLMRequest, LLMResponse

_graph_registry: Dict[str, Type[BaseAgentGraph]] = {}


def register(agent_name: str):
    def deco(sub):
        _graph_registry[agent_name] = sub
        return sub
    return deco


class AgentModule(RolloutModule):
    def __init__(self, name: str, args=None, replica_id: int = 0):
        super().__init__(name, args, replica_id)
        self.agent_factory: Dict[str, BaseAgentGraph] = {}

    def build_agent_graph(self, agent_name: str, agent_cfg_path=None) -> BaseAgentGraph:
        if agent_name not in _graph_registry:
            from . import examples  # noqa: F401  (registers the bundled graphs)
        assert agent_name in _graph_registry, f"no agent graph registered as {agent_name!r}"
        cfg = None
        if agent_cfg_path:
            from chatlearn_b200.configs.conf import load_yaml
            cfg = load_yaml(agent_cfg_path)
        g = _graph_registry[agent_name](agent_name=agent_name, cfg=cfg, llm=self, tokenizer=self.tokenizer,
                                        processor=getattr(self, "processor", None),
                                        model_type=getattr(self.runtime_args, "model_type", "llm"))
        if self.engine.vision is not None and getattr(g, "chatmodel", None) is not None:
            g.chatmodel.vision = {"image_token_id": self.arch.image_token_id, "video_token_id": self.arch.video_token_id,
                                  "merge_size": self.engine.vision.arch.spatial_merge_size}
        self.agent_factory[agent_name] = g
        return g

    # ---- one batched engine call for all waiting trajectories ----
    def _answer(self, reqs: List[LLMRequest], is_eval: bool) -> List[LLMResponse]:
        ma = self.module_args
        base = self._sampling_params(is_eval, ma.max_response_tokens_length)
        sps, budgets = [], []
        for r in reqs:
            over = {k: v for k, v in r.sampling_params.items() if hasattr(base, k)}
            sp = SamplingParams(**{**base.__dict__, **over})
            mx = int(r.sampling_params.get("max_new_tokens", sp.max_tokens))
            budgets.append(max(0, min(mx, ma.seq_length - len(r.token_ids))))
            sps.append(sp)
        mm = [r.mm for r in reqs] if self.engine.vision is not None and any(r.mm is not None for r in reqs) else None
        seqs = self.engine.generate([r.token_ids for r in reqs], sps, max_new_tokens=budgets, mm_inputs=mm)
        return [LLMResponse(list(q.output), list(q.logprobs), q.finish_reason) for q in seqs]

    def _sync_objects(self, objs):
        """Broadcast from the replica's first tensor-parallel rank."""
        import torch.distributed as dist
        box = [objs]
        dist.broadcast_object_list(box, src=self.tp_group.ranks[0], group=self.tp_group.pg)
        return box[0]

    def _request_args(self, r: LLMRequest, base: SamplingParams):
        ma = self.module_args
        over = {k: v for k, v in r.sampling_params.items() if hasattr(base, k)}
        sp = SamplingParams(**{**base.__dict__, **over})
        mx = int(r.sampling_params.get("max_new_tokens", sp.max_tokens))
        return sp, max(0, min(mx, ma.seq_length - len(r.token_ids)))

    def _run_continuous(self, gens, waiting, done, is_eval: bool, multi: bool, lead: bool):
        """Open-session scheduling: ``waiting`` holds the first request of every trajectory (on the lead rank)."""
        base = self._sampling_params(is_eval, self.module_args.max_response_tokens_length)
        with_images = self.engine.vision is not None
        sess = self.engine.open_session()
        owner: Dict[int, int] = {}                    # request id -> trajectory
        fresh = [(i, waiting[i]) for i in sorted(waiting)] if lead else []
        self.agent_stats = {"requests": 0, "engine_steps": 0, "joined_running_batch": 0}
        while True:
            if multi:
                # one small broadcast per step tells the other ranks whether requests follow
                import torch.distributed as dist
                n = torch.tensor([len(fresh)], dtype=torch.int32, device=self.engine.device)
                dist.broadcast(n, src=self.tp_group.ranks[0], group=self.tp_group.pg)
                fresh = self._sync_objects(fresh if lead else None) if int(n.item()) else []
            for i, r in fresh:
                sp, budget = self._request_args(r, base)
                if sess.sched.running:
                    self.agent_stats["joined_running_batch"] += 1
                seq = sess.submit(r.token_ids, sp, budget, r.mm if with_images else None)
                owner[seq.req_id] = i
                self.agent_stats["requests"] += 1
            finished = sess.poll()
            if finished is None:
                break
            self.agent_stats["engine_steps"] += 1
            fresh = []
            for q in finished:
                i = owner.pop(q.req_id)
                if not lead:
                    continue
                try:
                    fresh.append((i, gens[i].send(LLMResponse(list(q.output), list(q.logprobs), q.finish_reason))))
                except StopIteration as e:
                    done[i] = e.value
        sess.close()

    def run_trajectories(self, data_list: List[Dict], is_eval: bool = False) -> List[AgentGraphOutput]:
        ma = self.module_args
        sampling = {"max_new_tokens": ma.max_response_tokens_length}
        multi = self.tp_group is not None and self.tp_group.size > 1
        lead = not multi or self.tp_group.rank == 0
        gens, waiting, done = [], {}, {}
        if lead:
            # only the replica's first rank runs the graphs (and therefore the tools)
            for i, q in enumerate(data_list):
                assert q.get("agent_name"), "agent tasks need an agent_name field in the dataset"
                name = q["agent_name"]
                graph = self.agent_factory.get(name) or self.build_agent_graph(name, q.get("agent_cfg_path"))
                gens.append(graph.run(sampling_params=dict(sampling), **q))
            for i, g in enumerate(gens):
                try:
                    waiting[i] = next(g)
                except StopIteration as e:
                    done[i] = e.value
        if str(getattr(ma, "agent_scheduling", "continuous")) == "continuous":
            self._run_continuous(gens, waiting, done, is_eval, multi, lead)
            waiting = {}
        while True:
            order = sorted(waiting)
            reqs = self._sync_objects([waiting[i] for i in order] if lead else None) if multi \
                else [waiting[i] for i in order]
            if not reqs:
                break
            resps = self._answer(reqs, is_eval)
            if lead:
                nxt = {}
                for i, r in zip(order, resps):
                    try:
                        nxt[i] = gens[i].send(r)
                    except StopIteration as e:
                        done[i] = e.value
                waiting = nxt
        outs = [done[i] for i in range(len(gens))] if lead else None
        return self._sync_objects(outs) if multi else outs

    def generate_per_request(self, query: Dict, is_eval: bool = False) -> AgentGraphOutput:
        return self.run_trajectories([query], is_eval)[0]

    def postprocess_func(self, outputs: List[AgentGraphOutput], data_list: List[Dict]) -> List[Dict]:
        res = []
        for o, d in zip(outputs, data_list):
            r = dict(d)
            n_prompt = len(o.prompt_ids)
            r.update({
                "loss_mask": torch.tensor(o.loss_mask, dtype=torch.long),
                "prompt_token_ids": list(o.prompt_ids),
                "all_tokens": torch.tensor(o.all_token_ids, dtype=torch.long),
                "response_token_length": len(o.all_token_ids) - n_prompt,
                "prompt_token_length": n_prompt,
                "all_token_length": len(o.all_token_ids),
                "str_outputs": o.str_output,
                "num_turns": o.num_turns,
                "pixel_values": o.pixel_values, "image_grid_thw": o.image_grid_thw,
                "visual_time_steps": o.visual_time_steps,
                "attention_mask": o.attention_mask,
            })
            if o.response_logprobs is not None:
                r["rollout_logprobs"] = torch.tensor(o.response_logprobs, dtype=torch.float32)
            res.append(r)
        return res

    def forward_step(self, data_list: List[Dict], iteration: int = 0, is_eval: bool = False, **kw):
        outs = self.run_trajectories(data_list, is_eval)
        res = self.postprocess_func(outs, data_list)
        if not is_eval and res:
            lens = torch.tensor([o["response_token_length"] for o in res], dtype=torch.float32)
            self._metric_list.append({
                "response_length": lens.mean().item(), "response_length_max": lens.max().item(),
                "response_clip_ratio": (lens >= self.module_args.max_response_tokens_length).float().mean().item(),
                "num_turns": sum(o["num_turns"] for o in res) / len(res)})
        return res
