"""Math agent whose tool checks a proposed answer against the ground truth
(chatlearn/models/agent/examples/math_eval_agent_graph.py:33-167)."""
from chatlearn_b200.models.agent.agent_module import register
from chatlearn_b200.utils.rule_reward_score.math import is_equiv
from .tool_agent import ToolLoopAgentGraph


@register("matheval_agent")
class MathEvalAgentGraph(ToolLoopAgentGraph):
    def tools(self):
        def mathlighteval_reward(answer: str, **kwargs):
            """A tool for calculating the reward of mathlighteval."""
            return "The answer is correct." if is_equiv(answer, kwargs["ground_truth"]) else "The answer is wrong."

        return [mathlighteval_reward]
