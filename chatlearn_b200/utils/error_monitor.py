"""Job-wide error signalling.

Parity: chatlearn/utils/error_monitor.py:25-76.  The reference keeps a named
``ErrorSignalActor`` in Ray that workers set on failure and an ``ErrorMonitor`` actor
that polls it every two seconds and kills all actors.  Without Ray the shared state is
a directory (``CLB200_ERROR_DIR``, created by the job supervisor in
``launcher/local.py``): a failing rank drops a ``rank<r>.err`` file there
(``runtime/decorator.py: report_error``), every rank can ask ``ErrorSignal.is_set()``
between steps, and the supervisor ends the job when a file appears.
"""
import os
import threading
from typing import Callable, List, Optional


class ErrorSignal:
    def __init__(self, directory: Optional[str] = None):
        self.dir = directory or os.environ.get("CLB200_ERROR_DIR")

    def set(self, err_msg: str = ""):
        if not self.dir:
            return
        os.makedirs(self.dir, exist_ok=True)
        with open(os.path.join(self.dir, f"rank{os.environ.get('RANK', '0')}.err"), "a", encoding="utf-8") as f:
            f.write(err_msg + "\n")

    def reports(self) -> List[str]:
        if not self.dir or not os.path.isdir(self.dir):
            return []
        return sorted(f for f in os.listdir(self.dir) if f.endswith(".err"))

    def is_set(self) -> bool:
        return bool(self.reports())

    def error_msg(self) -> str:
        out = []
        for f in self.reports():
            with open(os.path.join(self.dir, f), encoding="utf-8") as fh:
                out.append(f"[{f[:-4]}] " + fh.read().strip())
        return "\n".join(out)


class ErrorMonitor:
    """Polls the signal from a daemon thread and calls ``on_error(message)`` once."""

    def __init__(self, signal: Optional[ErrorSignal] = None, on_error: Optional[Callable[[str], None]] = None,
                 interval_s: float = 2.0):
        self.signal = signal or ErrorSignal()
        self.on_error = on_error or (lambda msg: os._exit(1))
        self.interval = interval_s
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def monitor(self):
        def run():
            while not self._stop.is_set():
                if self.signal.is_set():
                    self.on_error(self.signal.error_msg())
                    return
                self._stop.wait(self.interval)
        self._thread = threading.Thread(target=run, daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
