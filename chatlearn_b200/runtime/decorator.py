"""Decorators around a role's compute methods.

Parity: chatlearn/runtime/decorator.py:29-166.  The reference wraps every exposed
method of every Ray actor: ``monitor_error`` reports an exception to a named
``ErrorSignalActor`` before re-raising, ``timeit`` times the call under the method's
name, ``compute_decorator`` fetches/merges the inputs, loops over generation batches,
switches train/eval mode and handles onload/offload.  In this runtime the executor
does the batching and residency (runtime/executor.py), so the decorators here cover
what remains per call: error reporting to the supervisor, timing, train/eval mode and
the iteration counter.  They are applied by ``BaseModule`` subclasses or by users
who expose extra flow functions.
"""
import functools
import os
import time
import traceback

from chatlearn_b200.utils.logger import logger


def report_error(where: str, exc: BaseException):
    """Make a failure visible to the job supervisor (launcher/local.py): one file per
    rank under ``CLB200_ERROR_DIR``; the supervisor ends the other ranks when one appears."""
    d = os.environ.get("CLB200_ERROR_DIR")
    text = f"{where}: {type(exc).__name__}: {exc}\n{traceback.format_exc()}"
    logger.error(f"catch exception ========= in {where}: {exc}")
    if d:
        try:
            os.makedirs(d, exist_ok=True)
            with open(os.path.join(d, f"rank{os.environ.get('RANK', '0')}.err"), "a") as f:
                f.write(text)
        except OSError:
            pass


def monitor_error(func=None):
    def deco(fn):
        @functools.wraps(fn)
        def inner(self, *args, **kwargs):
            try:
                return fn(self, *args, **kwargs)
            except Exception as e:
                report_error(f"{getattr(self, 'name', type(self).__name__)}.{fn.__name__}", e)
                raise
        return inner
    return deco(func) if callable(func) else deco


def timeit(name=None):
    def deco(fn):
        label = name or fn.__name__

        @functools.wraps(fn)
        def inner(self, *args, **kwargs):
            timers = getattr(self, "timers", None)
            if timers is None:
                t0 = time.perf_counter()
                try:
                    return fn(self, *args, **kwargs)
                finally:
                    logger.debug(f"{label}: {time.perf_counter() - t0:.3f} s")
            timers(label).start()
            try:
                return fn(self, *args, **kwargs)
            finally:
                timers(label).stop()
        return inner
    return deco


def compute_decorator(trainable: bool, rollout: bool = False):
    """Train/eval mode + iteration bookkeeping around a flow function."""
    def deco(fn):
        @functools.wraps(fn)
        def inner(self, data, iteration=0, **kwargs):
            (self.train if trainable else self.eval)()
            self._iteration = iteration
            out = fn(self, data, iteration, **kwargs)
            if trainable:
                self._train_iteration = getattr(self, "_train_iteration", 0) + 1
            return out
        inner.is_rollout = rollout
        return inner
    return deco
