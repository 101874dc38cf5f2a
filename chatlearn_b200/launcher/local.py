"""Local multi-process launcher with a supervisor.

The reference bootstraps a Ray cluster and relies on an ``ErrorMonitor`` actor
polling every 2 s plus ``ExitActor`` mailboxes to tear the job down when a
worker fails (chatlearn/utils/error_monitor.py:25-76,
chatlearn/launcher/dlc_utils.py:150-258).  Here the supervisor is the parent
process: it forks one rank per GPU (or CPU rank), watches exit codes and the
per-rank heartbeat files, and on the first failure or missed heartbeat terminates
the remaining ranks and re-raises, so a crashed or wedged rank never leaves the
others blocked in a collective.
"""
import os
import signal
import subprocess
import tempfile
import time
from typing import List, Optional

from chatlearn_b200.utils.utils import get_free_port


class RankFailure(RuntimeError):
    pass


def launch_local(cmd: List[str], nproc: int, cpu: bool = False, env: Optional[dict] = None,
                 heartbeat_timeout_s: float = 0.0, poll_s: float = 0.5,
                 stdout=None) -> int:
    """Run ``cmd`` as ``nproc`` ranks on this host; returns 0 or raises ``RankFailure``."""
    port = get_free_port()
    hb_dir = tempfile.mkdtemp(prefix="chatlearn_hb_")
    err_dir = os.path.join(hb_dir, "errors")      # ranks report caught exceptions here (runtime/decorator.py)
    procs = []
    for r in range(nproc):
        e = dict(os.environ)
        e.update(env or {})
        e.update(RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(nproc), LOCAL_WORLD_SIZE=str(nproc),
                 MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CHATLEARN_HEARTBEAT_DIR=hb_dir,
                 CLB200_ERROR_DIR=err_dir)
        if cpu:
            e["CHATLEARN_FORCE_CPU"] = "1"
        procs.append(subprocess.Popen(cmd, env=e, stdout=stdout, stderr=subprocess.STDOUT if stdout else None,
                                      start_new_session=True))
    failed = None
    try:
        while True:
            alive = 0
            for r, p in enumerate(procs):
                rc = p.poll()
                if rc is None:
                    alive += 1
                    if heartbeat_timeout_s > 0:
                        hb = os.path.join(hb_dir, f"rank{r}")
                        if os.path.exists(hb) and time.time() - os.path.getmtime(hb) > heartbeat_timeout_s:
                            failed = (r, "heartbeat timeout")
                elif rc != 0:
                    failed = (r, f"exit code {rc}")
            if not failed and os.path.isdir(err_dir):
                errs = sorted(os.listdir(err_dir))
                if errs:
                    with open(os.path.join(err_dir, errs[0]), encoding="utf-8") as f:
                        failed = (int(errs[0][4:-4]), "reported " + f.readline().strip())
            if failed or alive == 0:
                break
            time.sleep(poll_s)
    finally:
        if failed:
            for p in procs:
                if p.poll() is None:
                    try:
                        os.killpg(p.pid, signal.SIGTERM)   # exact process group we started
                    except ProcessLookupError:
                        pass
            deadline = time.time() + 10
            for p in procs:
                try:
                    p.wait(timeout=max(0.1, deadline - time.time()))
                except subprocess.TimeoutExpired:
                    try:
                        os.killpg(p.pid, signal.SIGKILL)
                    except ProcessLookupError:
                        pass
    if failed:
        raise RankFailure(f"rank {failed[0]} failed: {failed[1]}")
    return 0


class Heartbeat:
    """Touches ``$CHATLEARN_HEARTBEAT_DIR/rank{r}`` from a daemon thread."""

    def __init__(self, interval_s: float = 2.0):
        import threading
        self.dir = os.environ.get("CHATLEARN_HEARTBEAT_DIR")
        self.rank = int(os.environ.get("RANK", "0"))
        self.interval = interval_s
        self._stop = threading.Event()
        self._paused = threading.Event()
        self._thread = None
        if self.dir:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def _run(self):
        path = os.path.join(self.dir, f"rank{self.rank}")
        while not self._stop.is_set():
            if not self._paused.is_set():
                with open(path, "w", encoding="utf-8") as f:
                    f.write(str(time.time()))
            self._stop.wait(self.interval)

    def pause(self):
        """Stop beating without exiting (fault-injection tests: a wedged rank)."""
        self._paused.set()

    def stop(self):
        self._stop.set()
