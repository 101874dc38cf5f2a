"""SPMD executor of a traced model flow.

Parity: chatlearn/runtime/executor.py:62-463 (graph execution per level, DP
regrouping between producers and consumers of different data-parallel size,
onload/offload flags for colocated models) and chatlearn/runtime/decorator.py
(data fetch/merge, timers, consumed samples).  The reference drives Ray actors
through queues of object refs and ships every stage output through the object
store.  Here every rank runs the same loop: for each node, the ranks hosting the
node's model run it on their slice of the episode's sample list; the keys a node
added are then exchanged so that every rank holds the complete, identically
ordered list (only the delta travels, and not at all when consumer and producer
partition the data the same way).
"""
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from chatlearn_b200.runtime.model_flow import ModelFlow, ModelNode
from chatlearn_b200.utils.logger import logger
from chatlearn_b200.utils.trace import span
from chatlearn_b200.utils.utils import even_slice


def _world():
    return dist.get_world_size() if dist.is_initialized() else 1


def _rank():
    return dist.get_rank() if dist.is_initialized() else 0


def all_gather_objects(obj) -> List[Any]:
    if _world() == 1:
        return [obj]
    out = [None] * _world()
    dist.all_gather_object(out, obj)
    return out


class _TensorRef:
    """Stand-in for a tensor that travels on the tensor plane: (dtype, offset, shape) into the rank's flat buffer."""
    __slots__ = ("dtype", "off", "shape")

    def __init__(self, dtype, off, shape):
        self.dtype, self.off, self.shape = dtype, off, shape


_PLANE_MIN_ELEMS = 16


def gather_payloads(payload) -> List[Any]:
    """All-gather of per-rank payloads (nested dicts / lists / tuples of samples) in two planes: the tensors in
    them (token ids, per-token log-probs, ...) are concatenated per dtype into one flat buffer per rank and
    exchanged with a tensor collective, everything else (a few scalars and strings per sample, and the
    structure) is pickled.  The reference ships every stage output through Ray's object store
    (chatlearn/runtime/executor.py:245-330); here what is pickled does not grow with the sequence length."""
    if _world() == 1:
        return [payload]
    flats: Dict[torch.dtype, List[torch.Tensor]] = {}
    sizes: Dict[torch.dtype, int] = {}

    def strip(o):
        if torch.is_tensor(o):
            if o.device.type == "cpu" and o.numel() >= _PLANE_MIN_ELEMS and not o.is_sparse and o.layout == torch.strided:
                off = sizes.get(o.dtype, 0)
                flats.setdefault(o.dtype, []).append(o.detach().reshape(-1))
                sizes[o.dtype] = off + o.numel()
                return _TensorRef(o.dtype, off, tuple(o.shape))
            return o
        if isinstance(o, dict):
            return {k: strip(v) for k, v in o.items()}
        if isinstance(o, list):
            return [strip(v) for v in o]
        if isinstance(o, tuple):
            return tuple(strip(v) for v in o)
        return o

    meta = strip(payload)
    world = _world()
    metas = all_gather_objects((meta, {str(k): (k, v) for k, v in sizes.items()}))
    dtypes = {}
    for _, sz in metas:
        for name, (dt, n) in sz.items():
            dtypes[name] = (dt, max(n, dtypes.get(name, (dt, 0))[1]))
    gathered: Dict[torch.dtype, torch.Tensor] = {}
    cuda = dist.get_backend() == "nccl"
    for name in sorted(dtypes):                                # same order on every rank
        dt, width = dtypes[name]
        mine = torch.zeros(width, dtype=dt)
        if dt in flats:
            torch.cat(flats[dt], out=mine[:sizes[dt]])
        if cuda:
            from chatlearn_b200.utils import xfer
            dev = torch.device("cuda", torch.cuda.current_device())
            out = torch.empty(world * width, dtype=dt, device=dev)
            dist.all_gather_into_tensor(out, mine.to(dev, non_blocking=True))
            xfer.h2d_bytes += mine.numel() * mine.element_size()
            xfer.d2h_bytes += out.numel() * out.element_size()
            out = out.cpu()
        else:
            parts = [torch.empty(width, dtype=dt) for _ in range(world)]
            dist.all_gather(parts, mine)
            out = torch.cat(parts)
        gathered[dt] = out.view(world, width)

    def fill(o, r):
        if isinstance(o, _TensorRef):
            n = 1
            for d in o.shape:
                n *= d
            return gathered[o.dtype][r, o.off:o.off + n].view(o.shape).clone()
        if isinstance(o, dict):
            return {k: fill(v, r) for k, v in o.items()}
        if isinstance(o, list):
            return [fill(v, r) for v in o]
        if isinstance(o, tuple):
            return tuple(fill(v, r) for v in o)
        return o

    return [fill(m, r) for r, (m, _) in enumerate(metas)]


class Executor:
    def __init__(self, model_flow: Callable):
        self._flow_fn = model_flow
        self.models: List = []
        self.model_flow: Optional[ModelFlow] = None
        self.timers = None
        self.global_args = None
        self._metric_prefix = "executor"
        self._metric_list: List[Dict] = []
        self.is_eval = False

    # ------------------------------------------------------------------ wiring
    def set_timers(self, timers):
        self.timers = timers

    def update_models(self, models):
        """Keep the models this flow touches (found by tracing)."""
        flow = ModelFlow(models).trace(self._flow_fn)
        used = []
        for n in flow.model_nodes:
            if n.model not in used:
                used.append(n.model)
        self.models = used
        self.model_flow = flow
        return self

    def setup(self):
        if self.model_flow is None:
            raise RuntimeError("update_models() must be called before setup()")

    @property
    def first_node(self) -> ModelNode:
        return self.model_flow.flow_topology[0][0]

    def first_model(self):
        return self.first_node.model

    # ------------------------------------------------------------------ execution
    def _residency_flags(self, model, step: int, num_steps: int):
        """to_onload for the first step, to_offload for the last, only for colocated
        models that asked for memory to be freed (executor.py:396-403)."""
        fg = getattr(model, "residency_args", None) or getattr(model.module_args, "free_gpu_memory", None)
        wants = fg is not None and (fg.offload_weights or fg.free_grad_buffers or fg.offload_optimizer_states)
        on = model.is_colocate and wants
        return on and step == 0, on and step == num_steps - 1

    def _run_node(self, node: ModelNode, my_samples: List[Dict], iteration: int, kwargs: Dict) -> List[Dict]:
        """Run one node on this rank's slice in batches of generation_batch_size."""
        model = node.model
        fn = getattr(model, node.func_name)
        bs = int(getattr(model.module_args, "generation_batch_size", 0) or 0)
        if node.func_name == "train_step" or bs <= 0 or getattr(model, "whole_batch", False):
            bs = max(len(my_samples), 1)
        chunks = [my_samples[s:s + bs] for s in range(0, len(my_samples), bs)] or [[]]
        out: List[Dict] = []
        tname = f"{model.name}.{node.func_name}"
        for i, chunk in enumerate(chunks):
            to_onload, to_offload = self._residency_flags(model, i, len(chunks))
            if to_onload:
                with span(f"{tname}.onload"):
                    if model.trainable and node.func_name != "train_step":
                        # scoring with the trainer needs its weights only
                        model.onload(to_build_grad_buffers=False, to_onload_optimizer_states=False)
                    else:
                        model.onload()
            model.timers(node.func_name).start()
            nvtx = bool(getattr(model.runtime_args, "nsys", False)) and torch.cuda.is_available()
            if nvtx:                       # named ranges for timeline profilers (decorator.py:58-59,71-72)
                torch.cuda.nvtx.range_push(tname)
            try:
                with span(f"{tname}.compute"):
                    res = fn(chunk, iteration, **kwargs) if node.func_name != "train_step" else fn(chunk, **kwargs)
            finally:
                if nvtx:
                    torch.cuda.nvtx.range_pop()
            model.timers(node.func_name).stop()
            if res is not None:
                out.extend(res)
            # rollout engines stay resident during evaluation (decorator.py:134-136)
            if to_offload and not (self.is_eval and node is self.first_node):
                with span(f"{tname}.offload"):
                    model.offload()
        if torch.cuda.is_available() and model.total_gpu > 0:
            logger.debug(f"{tname}: {torch.cuda.memory_allocated() / 2**30:.1f} GiB allocated, "
                         f"peak {torch.cuda.max_memory_allocated() / 2**30:.1f} GiB")
        return out

    def execute_flow(self, samples_by_rank_fn: Callable[[Any], List[Dict]], iteration: int,
                     is_eval: bool = False) -> Dict[ModelNode, List[Dict]]:
        """Run the traced flow once over an episode.

        ``samples_by_rank_fn(model)`` produces the *input* of the first node on the
        ranks that host it (this replica's prompts).  Returns, for every return
        node, the complete sample list in global order (identical on all ranks)."""
        self.is_eval = is_eval
        flow = self.model_flow
        results: Dict[ModelNode, List[Dict]] = {}
        partition: Dict[ModelNode, Any] = {}
        kwargs = {"is_eval": True} if is_eval else {}
        for level in flow.flow_topology:
            for node in level:
                model = node.model
                dp_size = model.data_parallel_size
                dp_rank = model.data_parallel_rank if model.is_member else -1
                ins = [n for n in node.input_nodes if n is not None]
                if not ins:
                    mine = samples_by_rank_fn(model) if model.is_member else []
                    start = None
                else:
                    merged = results[ins[0]]
                    for other in ins[1:]:
                        merged = [{**a, **b} for a, b in zip(merged, results[other])]
                    b = even_slice(len(merged), dp_size)
                    if model.is_member:
                        start = b[dp_rank]
                        mine = merged[b[dp_rank]:b[dp_rank + 1]]
                    else:
                        start, mine = None, []
                before = [dict(s) for s in mine] if ins else None
                with span(f"node {model.name}.{node.func_name}"):
                    out = self._run_node(node, mine, iteration, kwargs) if model.is_member else []
                if node.func_name == "train_step":
                    results[node] = []
                    continue
                # ---- exchange what this node produced ----
                lead = model.is_member and model.is_data_leader
                if not ins:
                    payload = (dp_rank, out) if lead else None
                    parts = [p for p in gather_payloads(payload) if p is not None]
                    parts.sort(key=lambda p: p[0])
                    results[node] = [s for _, lst in parts for s in lst]
                else:
                    if len(out) != len(mine):
                        # the node re-shaped the sample list (e.g. a manager that filters):
                        # ship whole samples
                        payload = (dp_rank, out, True) if lead else None
                    else:
                        delta = []
                        for o, b4 in zip(out, before):
                            delta.append({k: v for k, v in o.items()
                                          if k not in b4 or b4[k] is not v})
                        payload = (dp_rank, delta, False) if lead else None
                    parts = [p for p in gather_payloads(payload) if p is not None]
                    parts.sort(key=lambda p: p[0])
                    if any(p[2] for p in parts):
                        results[node] = [s for _, lst, _ in parts for s in lst]
                    else:
                        full = [dict(s) for s in merged]
                        bnd = even_slice(len(full), dp_size)
                        for r, delta, _ in parts:
                            for j, d in enumerate(delta):
                                full[bnd[r] + j].update(d)
                        results[node] = full
                # a role may re-order the complete list (same code on every rank)
                hook = getattr(model, "post_gather", None)
                if hook is not None:
                    results[node] = hook(results[node], node.func_name)
        return {n: results[n] for n in flow.return_nodes}

    # ------------------------------------------------------------------ metrics
    def get_and_clear_metrics(self):
        from chatlearn_b200.utils.utils import map_reduce_metrics
        if not self._metric_list:
            return self._metric_prefix, {}
        m = map_reduce_metrics(self._metric_list)
        self._metric_list = []
        return self._metric_prefix, m
