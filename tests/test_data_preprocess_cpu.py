import json

from chatlearn_b200.data.data import read_data_path_list
from chatlearn_b200.data.data_preprocess import gsm8k, gsm8k_agent, math_lighteval
from chatlearn_b200.data.data_preprocess.common import run_converter


def test_gsm8k_roundtrip(tmp_path):
    src = tmp_path / "raw" / "main"
    src.mkdir(parents=True)
    rows = [{"question": "1+1?", "answer": "easy\n#### 2"}, {"question": "big", "answer": "x\n#### 1,234"}]
    import pyarrow as pa
    import pyarrow.parquet as pq
    pq.write_table(pa.Table.from_pylist(rows), src / "train-00000.parquet")
    (src / "test.jsonl").write_text("\n".join(json.dumps(r) for r in rows[:1]))
    out = run_converter("", str(tmp_path / "out"), gsm8k.convert, argv=["--input_dir", str(tmp_path / "raw"), "--local_dir", str(tmp_path / "out")])
    assert out["train"][1] == 2 and out["test"][1] == 1
    data = read_data_path_list([out["train"][0]])[0]
    assert data[1]["reward_model"]["ground_truth"] == "1234" and data[0]["prompt"][0]["role"] == "user"
    assert "\\boxed{}" in data[0]["prompt"][0]["content"]
    a = gsm8k_agent.convert(dict(rows[0]), "train", 0)
    assert a["agent_name"] == "mathcode_agent" and a["prompt"][0]["role"] == "system"


def test_math_lighteval_extracts_last_box():
    ex = {"problem": "p", "solution": "so \\boxed{1} then \\boxed{\\frac{1}{2}}", "level": "3", "type": "alg"}
    r = math_lighteval.convert(ex, "train", 5)
    assert r["reward_model"]["ground_truth"] == "\\frac{1}{2}" and r["extra_info"]["index"] == 5
    assert math_lighteval.convert({"problem": "p", "solution": "no box"}, "train", 0) is None
