"""The parts of bench.py's contract that need no GPU: the reference arm's line, the baseline ratio, the
rollout / trainer agreement read-out, and the command line."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_one_unavailable_line_and_exits_zero():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                        "--warmup", "3"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]


def test_baseline_ratio_only_for_the_recorded_configuration(monkeypatch):
    b = _bench()
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = b.parse()
    rec = json.load(open(os.path.join(ROOT, "baseline", "library_baseline.json")))
    base = rec["runs"]["1"]["value"]
    assert abs(b.vs_baseline(1, 2 * base, args) - 2.0) < 1e-3
    assert b.vs_baseline(8, 10.0, args) is None                       # no library record at eight GPUs
    args.max_response = 4096
    assert b.vs_baseline(1, 2 * base, args) is None                   # another configuration: nothing to divide by
    args.max_response = 2048
    args.impl = "library"
    assert b.vs_baseline(1, 2 * base, args) is None


def test_agreement_metric_is_read_from_the_run_metrics(tmp_path):
    b = _bench()
    with open(tmp_path / "metrics.jsonl", "w") as f:
        for v in (0.5, 0.04, 0.06):
            f.write(json.dumps({"policy_trainer/rollout_logprob_abs_diff": v, "policy_trainer/rollout_logprob_abs_diff_max": 9.0}) + "\n")
    assert abs(b.rollout_trainer_diff(str(tmp_path), 2) - 0.05) < 1e-9       # the timed episodes are the last ones
    assert b.rollout_trainer_diff(str(tmp_path / "missing"), 2) is None


def test_defaults_finish_within_minutes(monkeypatch):
    b = _bench()
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    a = b.parse()
    assert a.gpus == 1 and a.warmup >= 3 and a.steps >= 1 and a.time_budget <= 800 and a.rollout_tp == 1
