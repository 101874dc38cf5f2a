"""The model/tools loop shared by the bundled agents.

``agent`` (a model turn) → if the turn asked for tools and the turn / token budgets
allow: ``tools`` (run them, append their answers) → ``agent`` …  (the shape of
chatlearn/models/agent/examples/math_code_agent_graph.py:34-169).
"""
import copy
from typing import Any, Callable, Dict, List

from chatlearn_b200.models.agent.base_agent_graph import END, BaseAgentGraph, StateGraph
from chatlearn_b200.models.agent.chat_model import ToolMessage


def _cfg(cfg, key, default):
    if cfg is None:
        return default
    v = cfg.get(key, default) if isinstance(cfg, dict) else getattr(cfg, key, default)
    return default if v is None else v


class ToolLoopAgentGraph(BaseAgentGraph):
    """Subclasses provide ``tools()``; tool functions may take ``**kwargs`` to receive the
    query's extra fields (for example ``ground_truth``), which are never shown to the model."""

    def __init__(self, agent_name, cfg=None, llm=None, tokenizer=None, processor=None, **kwargs):
        super().__init__(agent_name, cfg, llm, tokenizer, processor, **kwargs)
        self.max_ai_message_turn = int(_cfg(cfg, "max_ai_message_turn", 4))
        self.max_total_token_length = int(_cfg(cfg, "max_total_token_length", 8192))
        self.build_graph()

    def tools(self) -> List[Callable]:
        raise NotImplementedError

    def build_graph(self):
        super().build_graph()
        tools = self.tools()
        by_name = {t.__name__: t for t in tools}
        self.chatmodel = self.chatmodel.bind_tools(tools)

        def call_model(state, config):
            c = config["configurable"]
            mm = {"pixel_values": c.get("pixel_values"), "image_grid_thw": c.get("image_grid_thw"),
                  "visual_time_steps": c.get("visual_time_steps")} if c.get("pixel_values") is not None else None
            msg = yield from c["chat_model"].invoke(state["messages"], c["sampling_params"], mm)
            return {"messages": [msg]}

        def tool_node(state, config):
            extra = {k: v for k, v in config["configurable"].items()
                     if k not in ("chat_model", "sampling_params", "pixel_values", "image_grid_thw", "visual_time_steps")}
            outs = []
            for call in state["messages"][-1].tool_calls:
                args = copy.deepcopy(call["args"])
                try:
                    fn = by_name[call["name"]]
                    import inspect
                    takes_kw = any(p.kind == p.VAR_KEYWORD for p in inspect.signature(fn).parameters.values())
                    text = fn(**args, **(extra if takes_kw else {}))
                except Exception:  # unknown tool, bad arguments, tool failure: the model is told, the rollout goes on
                    text = "tool execute error"
                outs.append(ToolMessage(content=str(text), name=call["name"], tool_call_id=call["id"]))
            return {"messages": outs}

        def should_continue(state):
            msgs = state["messages"]
            turns = sum(1 for m in msgs if m.type == "ai")
            total = max((len(m.response_metadata["loss_mask"]) for m in msgs if m.type == "ai"), default=0)
            if not msgs[-1].tool_calls or turns >= self.max_ai_message_turn or total >= self.max_total_token_length:
                return "end"
            return "continue"

        g = StateGraph()
        g.add_node("agent", call_model)
        g.add_node("tools", tool_node)
        g.set_entry_point("agent")
        g.add_conditional_edges("agent", should_continue, {"continue": "tools", "end": END})
        g.add_edge("tools", "agent")
        self.graph = g.compile()

    def run(self, messages=None, sampling_params: Dict[str, Any] = None, **query):
        extra = {k: query[k] for k in ("ground_truth", "data_source", "pixel_values", "image_grid_thw",
                                       "visual_time_steps") if k in query}
        out = yield from self.default_run(messages, sampling_params or {}, **extra)
        return out
