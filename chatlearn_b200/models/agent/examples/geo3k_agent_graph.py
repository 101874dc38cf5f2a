"""Geometry3K agent: the model may ask a checker whether its boxed answer is right
(chatlearn/models/agent/examples/geo3k_agent_graph.py:33-171).  Images ride on the
query (``pixel_values`` / ``image_grid_thw`` prepared by the vision prompt pipeline)."""
from chatlearn_b200.models.agent.agent_module import register
from chatlearn_b200.utils.rule_reward_score.geo3k import acc_reward
from .tool_agent import ToolLoopAgentGraph


@register("geo3k_agent")
class Geo3kAgentGraph(ToolLoopAgentGraph):
    def tools(self):
        def geo3k_reward(answer: str, **kwargs):
            """A tool for checking an answer of a geometry problem."""
            ok = acc_reward(f"\\boxed{{{answer}}}", kwargs["ground_truth"]) > 0
            return "The answer is correct." if ok else "The answer is wrong."

        return [geo3k_reward]

    def run(self, messages=None, sampling_params=None, **query):
        out = yield from super().run(messages, sampling_params, **query)
        out.pixel_values, out.image_grid_thw = query.get("pixel_values"), query.get("image_grid_thw")
        out.visual_time_steps = query.get("visual_time_steps")
        return out
