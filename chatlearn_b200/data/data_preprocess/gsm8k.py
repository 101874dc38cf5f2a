"""GSM8K → prompt records (chatlearn/data/data_preprocess/gsm8k.py).
``python -m chatlearn_b200.data.data_preprocess.gsm8k --input_dir dataset/gsm8k --local_dir dataset/gsm8k``"""
import re

from .common import BOXED, record, run_converter

DATA_SOURCE = "openai/gsm8k"


def extract_solution(answer: str) -> str:
    m = re.search(r"#### (\-?[0-9\.\,]+)", answer)
    assert m is not None, "GSM8K answers end with '#### <number>'"
    return m.group(1).replace(",", "")


def convert(ex, split, idx):
    q, a = ex["question"], ex["answer"]
    return record(DATA_SOURCE, [{"role": "user", "content": q + " " + BOXED}], extract_solution(a), split, idx,
                  extra={"answer": a, "question": q})


if __name__ == "__main__":
    run_converter(__doc__, "~/data/gsm8k", convert)
