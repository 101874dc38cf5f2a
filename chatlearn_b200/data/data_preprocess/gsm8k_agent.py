"""GSM8K for the code-interpreter agent (chatlearn/data/data_preprocess/gsm8k_agent.py)."""
from .common import BOXED, CODE_AGENT_SYSTEM, record, run_converter
from .gsm8k import DATA_SOURCE, extract_solution


def convert(ex, split, idx):
    q, a = ex["question"], ex["answer"]
    msgs = [{"role": "system", "content": CODE_AGENT_SYSTEM}, {"role": "user", "content": q + " " + BOXED}]
    return record(DATA_SOURCE, msgs, extract_solution(a), split, idx, extra={"answer": a, "question": q},
                  agent_name="mathcode_agent", agent_cfg_path="template/agent/math_eval.yaml")


if __name__ == "__main__":
    run_converter(__doc__, "~/data/gsm8k", convert, suffix="_agent")
