import os

import pytest

from chatlearn_b200.runtime.decorator import compute_decorator, monitor_error, timeit
from chatlearn_b200.utils.timer import Timers


class Role:
    name = "r"

    def __init__(self):
        self._t = Timers()
        self.mode = None

    def timers(self, n):
        return self._t(n)

    def train(self):
        self.mode = "train"

    def eval(self):
        self.mode = "eval"

    @monitor_error()
    @timeit()
    def boom(self):
        raise ValueError("x")

    @compute_decorator(trainable=True)
    def train_step(self, data, iteration=0):
        return len(data)


def test_error_is_reported_and_reraised(tmp_path, monkeypatch):
    monkeypatch.setenv("CLB200_ERROR_DIR", str(tmp_path))
    monkeypatch.setenv("RANK", "3")
    with pytest.raises(ValueError):
        Role().boom()
    assert "ValueError" in open(os.path.join(tmp_path, "rank3.err")).read()


def test_compute_decorator_sets_mode_and_counts():
    r = Role()
    assert r.train_step([1, 2], 7) == 2 and r.mode == "train" and r._iteration == 7 and r._train_iteration == 1


def test_error_signal_and_monitor(tmp_path, monkeypatch):
    import time
    from chatlearn_b200.utils.error_monitor import ErrorMonitor, ErrorSignal
    monkeypatch.setenv("RANK", "1")
    sig = ErrorSignal(str(tmp_path / "errs"))
    assert not sig.is_set()
    seen = []
    mon = ErrorMonitor(sig, on_error=seen.append, interval_s=0.05).monitor()
    sig.set("policy.forward_step: ValueError: x")
    for _ in range(100):
        if seen:
            break
        time.sleep(0.02)
    mon.stop()
    assert seen and "rank1" in seen[0] and "ValueError" in seen[0]


def test_log_monitor_tails_and_collects_errors(tmp_path):
    from chatlearn_b200.utils.log_monitor import LogMonitor
    (tmp_path / "rank0.log").write_text("hello\n")
    out = []
    lm = LogMonitor(str(tmp_path), sink=out.append)
    assert lm.poll() == 1 and out == ["(rank0) hello"]
    with open(tmp_path / "rank0.log", "a") as f:
        f.write("RuntimeError: CUDA error: boom\n")
    (tmp_path / "rank1.log").write_text("fine\n")
    assert lm.poll() == 2 and len(lm.errors) == 1 and "(rank0)" in lm.errors[0]
