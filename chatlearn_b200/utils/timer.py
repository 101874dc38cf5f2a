"""Named timers.

Parity: chatlearn/utils/timer.py:35-141 (``_Timer`` / ``Timers.log``).  The
reference brackets every start/stop with ``torch.cuda.synchronize()``; here a
timer records CUDA events on the current stream when a GPU is present and
resolves them lazily, so timing a phase does not serialise the device.  Host
wall time is kept as the CPU fallback.
"""
import time

import torch


class _Timer:
    def __init__(self, name, device_timing=True):
        self.name = name
        self._elapsed = 0.0
        self._started = False
        self._t0 = 0.0
        self._count = 0
        self._device = bool(device_timing and torch.cuda.is_available())
        self._pending = []  # (start_event, stop_event)
        self._ev0 = None

    def start(self):
        assert not self._started, f"timer {self.name} already started"
        if self._device:
            self._ev0 = torch.cuda.Event(enable_timing=True)
            self._ev0.record()
        self._t0 = time.perf_counter()
        self._started = True

    def stop(self):
        assert self._started, f"timer {self.name} not started"
        if self._device:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            self._pending.append((self._ev0, ev1, time.perf_counter() - self._t0))
        else:
            self._elapsed += time.perf_counter() - self._t0
        self._count += 1
        self._started = False

    def _resolve(self):
        if self._pending:
            for ev0, ev1, host in self._pending:
                ev1.synchronize()
                # device span and host span both bound the phase; the larger is
                # the true duration (host work with an idle device, or queued
                # device work after the host returned)
                self._elapsed += max(ev0.elapsed_time(ev1) / 1e3, host)
            self._pending = []

    def reset(self):
        self._pending = []
        self._elapsed = 0.0
        self._count = 0
        self._started = False

    def elapsed(self, reset=True):
        was = self._started
        if was:
            self.stop()
        self._resolve()
        out = self._elapsed
        if reset:
            self.reset()
        if was:
            self.start()
        return out

    @property
    def count(self):
        return self._count


class Timers:
    """Group of named timers: ``timers("train").start()``."""

    def __init__(self, device_timing=True):
        self.timers = {}
        self._device_timing = device_timing

    def __call__(self, name):
        if name not in self.timers:
            self.timers[name] = _Timer(name, self._device_timing)
        return self.timers[name]

    def names(self):
        return list(self.timers)

    def log(self, names=None, normalizer=1.0, reset=True, return_dict=False, e2e_cost=None):
        names = names if names is not None else self.names()
        out = {}
        for n in names:
            if n in self.timers:
                out[n] = self.timers[n].elapsed(reset=reset) / normalizer
        if return_dict:
            return out
        s = "time (s)"
        for n, v in out.items():
            s += f" | {n}: {v:.3f}"
        if e2e_cost is not None:
            s += f" | e2e: {e2e_cost:.3f}"
        return s
