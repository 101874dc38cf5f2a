"""Follow per-rank log files and surface their lines in one place.

Parity: chatlearn/utils/log_monitor.py (the reference tails Ray's worker log files and
republishes them with an actor prefix).  Here ranks launched by ``launcher/local.py``
can write to ``<log_dir>/rank<r>.log``; ``LogMonitor`` tails those files from a daemon
thread and forwards new lines, prefixed with the rank, to a sink (stdout by default).
Lines that look like errors are kept in ``errors`` for a final summary.
"""
import glob
import os
import re
import sys
import threading
from typing import Callable, Dict, List, Optional

_ERR = re.compile(r"Traceback|Error|CUDA error|NCCL WARN|Segmentation fault", re.I)


class LogMonitor:
    def __init__(self, log_dir: str, pattern: str = "rank*.log", sink: Optional[Callable[[str], None]] = None,
                 interval_s: float = 0.5):
        self.log_dir, self.pattern, self.interval = log_dir, pattern, interval_s
        self.sink = sink or (lambda line: (sys.stdout.write(line + "\n"), sys.stdout.flush()))
        self._pos: Dict[str, int] = {}
        self.errors: List[str] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def poll(self) -> int:
        """Forward everything written since the last call; returns the number of lines."""
        n = 0
        for path in sorted(glob.glob(os.path.join(self.log_dir, self.pattern))):
            tag = os.path.splitext(os.path.basename(path))[0]
            try:
                with open(path, "r", encoding="utf-8", errors="replace") as f:
                    f.seek(self._pos.get(path, 0))
                    chunk = f.read()
                    self._pos[path] = f.tell()
            except OSError:
                continue
            for line in chunk.splitlines():
                out = f"({tag}) {line}"
                if _ERR.search(line):
                    self.errors.append(out)
                self.sink(out)
                n += 1
        return n

    def start(self):
        def run():
            while not self._stop.is_set():
                self.poll()
                self._stop.wait(self.interval)
            self.poll()
        self._thread = threading.Thread(target=run, daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
