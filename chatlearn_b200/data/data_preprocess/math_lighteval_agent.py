"""MATH-lighteval for the answer-checking agent
(chatlearn/data/data_preprocess/math_lighteval_agent.py)."""
from chatlearn_b200.utils.rule_reward_score.math import last_boxed_only_string
from .common import BOXED, record, run_converter
from .math_lighteval import DATA_SOURCE, extract_solution

SYSTEM = ("You are a math expert. Solve the problem step by step. You may call the `mathlighteval_reward` tool with "
          "your candidate answer to learn whether it is correct. Put your final answer within \\boxed{}.")


def convert(ex, split, idx):
    q, sol = ex["problem"], ex["solution"]
    if last_boxed_only_string(sol) is None:
        return None
    msgs = [{"role": "system", "content": SYSTEM}, {"role": "user", "content": q + " " + BOXED}]
    return record(DATA_SOURCE, msgs, extract_solution(sol), split, idx,
                  agent_name="matheval_agent", agent_cfg_path="template/agent/math_eval.yaml")


if __name__ == "__main__":
    run_converter(__doc__, "~/data/math", convert, suffix="_agent")
