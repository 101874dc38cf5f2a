"""Shared pieces of the dataset converters.

Every converter turns a downloaded dataset directory (parquet / json / jsonl files,
one per split) into ``train.json`` and ``test.json`` in the record schema the prompt
pipeline reads: ``{data_source, prompt: [messages], ability, reward_model:
{style, ground_truth}, extra_info}`` plus ``agent_name`` / ``agent_cfg_path`` for
agent tasks (chatlearn/data/data_preprocess/*.py).  Files are read with pyarrow /
json directly, so no dataset hub client is needed.
"""
import argparse
import glob
import json
import os
from typing import Callable, Dict, Iterable, List, Optional

BOXED = "Let's think step by step and output the final answer within \\boxed{}."

CODE_AGENT_SYSTEM = (
    "You are a math expert. You are given a question and you need to solve it step by step. "
    "You can write and execute Python code to perform calculation or verify your answer. "
    "You should print the result at the end of Python code. "
    "You should use the `execute_python` tool to execute Python code. "
    "Put your final answer within \\boxed{}.")


def read_split(input_dir: str, split: str) -> List[Dict]:
    """Rows of the files of ``input_dir`` (searched recursively) whose name contains ``split``."""
    rows: List[Dict] = []
    pats = [f"**/*{split}*.parquet", f"**/*{split}*.jsonl", f"**/*{split}*.json"]
    files = sorted({f for p in pats for f in glob.glob(os.path.join(os.path.expanduser(input_dir), p), recursive=True)})
    for f in files:
        if f.endswith(".parquet"):
            import pyarrow.parquet as pq
            rows.extend(pq.read_table(f).to_pylist())
        elif f.endswith(".jsonl"):
            rows.extend(json.loads(x) for x in open(f) if x.strip())
        else:
            txt = open(f).read().strip()
            rows.extend(json.loads(txt) if txt.startswith("[") else [json.loads(x) for x in txt.splitlines() if x.strip()])
    return rows


def write_json_lines(rows: Iterable[Dict], path: str):
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")


def record(data_source: str, messages: List[Dict], ground_truth, split: str, idx: int, ability: str = "math",
           extra: Optional[Dict] = None, agent_name: Optional[str] = None, agent_cfg_path: Optional[str] = None) -> Dict:
    r = {"data_source": data_source, "prompt": messages, "ability": ability,
         "reward_model": {"style": "rule", "ground_truth": ground_truth},
         "extra_info": {"split": split, "index": idx, **(extra or {})}}
    if agent_name:
        r["agent_name"], r["agent_cfg_path"] = agent_name, agent_cfg_path
    return r


def run_converter(description: str, default_out: str, convert: Callable[[Dict, str, int], Optional[Dict]],
                  suffix: str = "", argv=None):
    ap = argparse.ArgumentParser(description=description)
    ap.add_argument("--input_dir", required=True, help="directory holding the downloaded dataset files")
    ap.add_argument("--local_dir", default=default_out, help="where train/test json files are written")
    args = ap.parse_args(argv)
    out = {}
    for split in ("train", "test"):
        rows = [convert(dict(ex), split, i) for i, ex in enumerate(read_split(args.input_dir, split))]
        rows = [r for r in rows if r is not None]
        path = os.path.join(os.path.expanduser(args.local_dir), f"{split}{suffix}.json")
        write_json_lines(rows, path)
        out[split] = (path, len(rows))
        print(f"{split}: {len(rows)} records -> {path}")
    return out
