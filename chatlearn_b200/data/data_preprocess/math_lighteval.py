"""MATH-lighteval → prompt records (chatlearn/data/data_preprocess/math_lighteval.py).  The
ground truth is the content of the last ``\\boxed{}`` of the reference solution."""
from chatlearn_b200.utils.rule_reward_score.math import last_boxed_only_string, remove_boxed
from .common import BOXED, record, run_converter

DATA_SOURCE = "DigitalLearningGmbH/MATH-lighteval"


def extract_solution(solution: str) -> str:
    return remove_boxed(last_boxed_only_string(solution))


def convert(ex, split, idx):
    q, sol = ex["problem"], ex["solution"]
    if last_boxed_only_string(sol) is None:
        return None
    return record(DATA_SOURCE, [{"role": "user", "content": q + " " + BOXED}], extract_solution(sol), split, idx,
                  extra={k: ex[k] for k in ("level", "type") if k in ex})


if __name__ == "__main__":
    run_converter(__doc__, "~/data/math", convert)
