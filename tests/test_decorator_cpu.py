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
