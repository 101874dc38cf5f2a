"""Dataflow graph of a user flow function, obtained by fake execution.

Parity: chatlearn/runtime/model_flow.py:29-255.  The flow function is called
once with every model method replaced by a recorder that returns placeholder
data; each call becomes a ``ModelNode`` whose inputs are the nodes that produced
its arguments.  Nodes are then levelled topologically.  ``ControlDependencies``
adds ordering edges between models with no data dependency.
"""
from typing import Callable, Dict, List, Optional, Sequence

from chatlearn_b200.utils import global_vars


class ControlDependencies:
    """``with ControlDependencies(out_a): model_b.forward_step(x)`` makes the
    call inside the block wait for the node that produced ``out_a``."""

    def __init__(self, dependencies):
        if not isinstance(dependencies, (list, tuple)):
            dependencies = [dependencies]
        self.dependencies = list(dependencies)

    def __enter__(self):
        global_vars.set_dependencies(self.dependencies)
        return self

    def __exit__(self, *exc):
        global_vars.reset_dependencies()
        return False


class DummyData:
    """Placeholder flowing through a traced function."""

    def __init__(self, from_node: Optional["ModelNode"] = None):
        self.from_node = from_node
        self.to_nodes: List["ModelNode"] = []


class ModelNode:
    def __init__(self, model, func_name: str):
        self.model = model
        self.name = model.name
        self.func_name = func_name
        self.input_nodes: List[Optional["ModelNode"]] = []
        self.output_nodes: List["ModelNode"] = []
        self.dependent_nodes: List["ModelNode"] = []     # control dependencies
        self.trainable = func_name in getattr(model, "trainable_funcs", []) or func_name == "train_step"
        self.out_data: Optional[DummyData] = None

    def add_input_node(self, node):
        self.input_nodes.append(node)
        if node is not None and self not in node.output_nodes:
            node.output_nodes.append(self)

    def __repr__(self):
        return f"<ModelNode {self.name}.{self.func_name}>"


class ModelFlow:
    def __init__(self, models: Sequence):
        self.models = list(models)
        self.model_nodes: List[ModelNode] = []
        self.return_nodes: List[ModelNode] = []
        self.flow_topology: List[List[ModelNode]] = []
        self.input_consumers: List[ModelNode] = []

    def trace(self, flow_fn: Callable, funcs_per_model: Optional[Dict[str, List[str]]] = None):
        """Run ``flow_fn`` with recorders in place of the model methods."""
        funcs_per_model = funcs_per_model or {}
        default = ["forward_step", "train_step", "eval_forward", "get_sample_for_rollout",
                   "post_process_rollout_results"]
        saved = []
        nodes: List[ModelNode] = []

        def recorder(model, fname):
            def fake(*args, **kwargs):
                node = ModelNode(model, fname)
                for a in args:
                    if isinstance(a, DummyData):
                        node.add_input_node(a.from_node)
                        a.to_nodes.append(node)
                        if a.from_node is None:
                            self.input_consumers.append(node)
                deps = global_vars.get_dependencies()
                if deps:
                    for d in deps:
                        if isinstance(d, DummyData) and d.from_node is not None:
                            node.dependent_nodes.append(d.from_node)
                out = DummyData(node)
                node.out_data = out
                nodes.append(node)
                return out
            return fake

        for m in self.models:
            names = set(default) | set(funcs_per_model.get(m.name, [])) | set(getattr(m, "call_funcs", []))
            for fname in names:
                if hasattr(m, fname):
                    saved.append((m, fname, m.__dict__.get(fname, None)))
                    setattr(m, fname, recorder(m, fname))
        try:
            ret = flow_fn(DummyData(None))
        finally:
            for m, fname, orig in saved:
                if orig is None:
                    try:
                        delattr(m, fname)
                    except AttributeError:
                        pass
                else:
                    setattr(m, fname, orig)
        if ret is None:
            rets = []
        elif isinstance(ret, (list, tuple)):
            rets = list(ret)
        else:
            rets = [ret]
        self.model_nodes = nodes
        self.return_nodes = [r.from_node for r in rets if isinstance(r, DummyData) and r.from_node]
        self.flow_topology = self.topological_sort()
        return self

    def topological_sort(self) -> List[List[ModelNode]]:
        """Levels: a node sits one level after its last data/control predecessor."""
        indeg = {n: 0 for n in self.model_nodes}
        succ: Dict[ModelNode, List[ModelNode]] = {n: [] for n in self.model_nodes}
        for n in self.model_nodes:
            preds = [p for p in n.input_nodes if p is not None] + n.dependent_nodes
            for p in set(preds):
                indeg[n] += 1
                succ[p].append(n)
        level = [n for n in self.model_nodes if indeg[n] == 0]
        out, seen = [], 0
        while level:
            out.append(level)
            seen += len(level)
            nxt = []
            for n in level:
                for s in succ[n]:
                    indeg[s] -= 1
                    if indeg[s] == 0:
                        nxt.append(s)
            level = nxt
        assert seen == len(self.model_nodes), "the model flow has a cycle"
        return out

    def linear_order(self) -> List[ModelNode]:
        return [n for lvl in self.flow_topology for n in lvl]
