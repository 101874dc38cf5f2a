"""Wall-clock span tracing of an episode.

``CLB200_TRACE=1`` turns it on: every ``span(name)`` synchronises the device on
entry and exit, so the recorded time is the time of the work inside it, and
``dump()`` logs the nested timeline (rank 0) and clears it.  Off (the default), a
span costs one dictionary lookup.  The reference has per-function timers only
(chatlearn/utils/timer.py); the nesting is what shows the gaps between them.
"""
import os
import time
from contextlib import contextmanager
from typing import List, Tuple

import torch

_ON = os.environ.get("CLB200_TRACE", "0") not in ("0", "")
_stack: List[str] = []
_events: List[Tuple[int, str, float]] = []


def enabled() -> bool:
    return _ON


def _sync():
    if torch.cuda.is_available():
        torch.cuda.synchronize()


@contextmanager
def span(name: str):
    if not _ON:
        yield
        return
    _sync()
    t0 = time.perf_counter()
    idx = len(_events)
    _events.append((len(_stack), name, 0.0))
    _stack.append(name)
    try:
        yield
    finally:
        _sync()
        _stack.pop()
        _events[idx] = (_events[idx][0], name, time.perf_counter() - t0)


def dump(log=None, min_s: float = 0.005) -> List[Tuple[int, str, float]]:
    ev = list(_events)
    _events.clear()
    if _ON and log is not None:
        lines = [f"{'  ' * d}{n}: {t:.3f}s" for d, n, t in ev if t >= min_s]
        log("trace\n" + "\n".join(lines))
    return ev
