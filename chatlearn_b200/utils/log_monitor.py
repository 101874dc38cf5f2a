"""Follow per-rank log files and surface their lines in one place.

Parity: chatlearn/utils/log_monitor.py (the reference tails Ray's worker log files and
republishes them with an actor prefix).  Here ranks launched by ``launcher/local.py``
can write to ``<log_dir>/rank<r>.log``; ``LogMonitor`` tails those files from a daemon
thread and forwards new lines, prefixed with the rank, to a sink (stdout by default).
Lines that look like errors are kept in ``errors`` for a final summary.

Several nodes: ``StoreLogPublisher`` is a sink that appends lines to a key-value store
(the launchers' ``TCPStore`` on node 0) under a per-node sequence, and ``StoreLogCollector``
on node 0 drains all nodes' sequences into its own sink, so one console shows the whole job
with ``(node<n>:rank<r>)`` prefixes, the way the reference's driver shows every actor's log.
Only error-like lines and a rate-limited sample of the rest travel unless ``everything`` is set.
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


class StoreLogPublisher:
    """Sink for ``LogMonitor`` on a worker node: appends lines to ``log/<node>/<seq>`` in a key-value store."""

    def __init__(self, store, node_rank: int, everything: bool = False, max_lines_per_s: float = 20.0):
        self.store, self.node, self.everything = store, node_rank, everything
        self.rate = max_lines_per_s
        self._seq = 0
        self._window, self._sent = 0, 0

    def __call__(self, line: str):
        import time
        if not (self.everything or _ERR.search(line)):
            w = int(time.time())
            if w != self._window:
                self._window, self._sent = w, 0
            if self._sent >= self.rate:
                return
            self._sent += 1
        self.store.set(f"log/{self.node}/{self._seq}", line)
        self._seq += 1
        self.store.set(f"log/{self.node}/n", str(self._seq))


class StoreLogCollector:
    """On node 0: forwards what the other nodes published, prefixed with the node."""

    def __init__(self, store, nnodes: int, sink: Optional[Callable[[str], None]] = None, interval_s: float = 0.5):
        self.store, self.nnodes, self.interval = store, nnodes, interval_s
        self.sink = sink or (lambda line: (sys.stdout.write(line + "\n"), sys.stdout.flush()))
        self._next = {n: 0 for n in range(nnodes)}
        self.errors: List[str] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def poll(self) -> int:
        got = 0
        for n in range(self.nnodes):
            key = f"log/{n}/n"
            try:
                if not self.store.check([key]):
                    continue
                upto = int(self.store.get(key).decode())
            except Exception:                       # the store went away with the job
                return got
            while self._next[n] < upto:
                line = self.store.get(f"log/{n}/{self._next[n]}").decode(errors="replace")
                self.store.delete_key(f"log/{n}/{self._next[n]}")
                self._next[n] += 1
                out = f"(node{n}:{line[1:]}" if line.startswith("(") else f"(node{n}) {line}"
                if _ERR.search(line):
                    self.errors.append(out)
                self.sink(out)
                got += 1
        return got

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
