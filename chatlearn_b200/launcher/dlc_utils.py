"""Multi-node bootstrap: one launcher per node starts that node's ranks and the launchers keep
watch over each other.

The reference starts a Ray cluster from the PAI-DLC job environment (``RANK`` = node index,
``WORLD_SIZE`` = node count, ``MASTER_ADDR``, ``CUSTOM_PORTS``), filters reserved ports, gives every
node an ``ExitActor`` mailbox and runs a ``StartExitListener`` thread so that worker nodes exit when
the head dies and remote errors are re-raised (chatlearn/launcher/dlc_utils.py:106-258).  Here there
is no Ray: the same environment is turned into a ``torch.distributed`` job (global rank = node
index x ranks per node + local rank), and the mailbox is a TCP key-value store served by node 0:

* a node whose rank fails (exit code, missed heartbeat, reported exception) posts the error;
* every launcher polls the mailbox and stops its ranks when another node posted an error;
* a launcher that cannot reach node 0 any more treats the head as dead and stops its ranks;
* node 0 keeps the store up until every node has reported that its ranks are finished.

``python -m chatlearn_b200.launcher.dlc_utils --nproc-per-node 8 -- python -m chatlearn_b200 grpo ...``
"""
import argparse
import os
import signal
import subprocess
import sys
import tempfile
import time
from dataclasses import dataclass, field
from datetime import timedelta
from typing import List, Optional

from chatlearn_b200.launcher.local import RankFailure
from chatlearn_b200.utils.utils import get_free_port


@dataclass
class NodeEnv:
    node_rank: int = 0
    nnodes: int = 1
    master_addr: str = "127.0.0.1"
    master_port: int = 29500
    reserved_ports: List[int] = field(default_factory=list)   # ports the platform assigned to this job


def _ports(text: str) -> List[int]:
    return [int(p) for p in text.replace(";", ",").split(",") if p.strip()]


def node_env(environ=None) -> NodeEnv:
    """Read the job description of a PAI-DLC / torchrun-style multi-node job."""
    e = os.environ if environ is None else environ
    nnodes = int(e.get("NNODES", e.get("WORLD_SIZE", "1")))
    node_rank = int(e.get("NODE_RANK", e.get("RANK", "0")))
    addr = e.get("MASTER_ADDR") or e.get("LOCAL_MASTER_ADDR") or "127.0.0.1"
    ports = _ports(e.get("CUSTOM_PORTS", ""))
    port = int(e.get("MASTER_PORT", ports[0] if ports else 29500))
    assert 0 <= node_rank < nnodes, f"node rank {node_rank} outside 0..{nnodes - 1}"
    return NodeEnv(node_rank, nnodes, addr, port, ports)


def get_free_ports(n: int, reserved: Optional[List[int]] = None, exclude=()) -> List[int]:
    """``n`` distinct usable ports: the platform's reserved ports first (those still free),
    then whatever the OS hands out."""
    import socket
    out = []
    for p in reserved or []:
        if p in exclude or p in out:
            continue
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            try:
                s.bind(("", p))
            except OSError:
                continue
        out.append(p)
        if len(out) == n:
            return out
    for _ in range(64 * n):
        p = get_free_port()
        if p not in out and p not in exclude:
            out.append(p)
        if len(out) == n:
            return out
    raise RuntimeError("not enough free ports")


class ExitMailbox:
    """Error mailbox and liveness record shared by the node launchers (key-value store on node 0)."""

    def __init__(self, env: NodeEnv, port: Optional[int] = None, timeout_s: float = 60.0):
        from torch.distributed import TCPStore
        self.env = env
        self.port = port if port is not None else env.master_port + 1
        self.store = TCPStore(env.master_addr, self.port, None, env.node_rank == 0,
                              timeout=timedelta(seconds=timeout_s), wait_for_workers=False)

    def post_error(self, text: str):
        if self.store.add("errors", 1) == 1:                 # the first report wins
            self.store.set("error", f"node {self.env.node_rank}: {text}")

    def error(self) -> Optional[str]:
        """The posted error, ``None`` if there is none; raises ``ConnectionError`` when node 0 is gone."""
        try:
            if not self.store.check(["error"]):
                return None
            return self.store.get("error").decode()
        except Exception as e:                               # the store's server side lives in node 0's launcher
            raise ConnectionError(f"head node unreachable: {e}") from e

    def done(self):
        self.store.add("done", 1)

    def all_done(self) -> bool:
        return self.store.add("done", 0) >= self.env.nnodes


def _stop(procs):
    for p in procs:
        if p.poll() is None:
            try:
                os.killpg(p.pid, signal.SIGTERM)            # exactly the process group started below
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


def launch_node(cmd: List[str], nproc_per_node: int, env: Optional[NodeEnv] = None, cpu: bool = False,
                extra_env: Optional[dict] = None, heartbeat_timeout_s: float = 0.0, poll_s: float = 0.5,
                mailbox_port: Optional[int] = None, drain_timeout_s: float = 600.0, stdout=None) -> int:
    """Run this node's share of the job; returns 0 or raises ``RankFailure`` (own rank failed, another
    node reported a failure, or the head node disappeared)."""
    env = env or node_env()
    box = ExitMailbox(env, mailbox_port)
    hb_dir = tempfile.mkdtemp(prefix="chatlearn_hb_")
    err_dir = os.path.join(hb_dir, "errors")
    world = env.nnodes * nproc_per_node
    procs = []
    for lr in range(nproc_per_node):
        e = dict(os.environ)
        e.update(extra_env or {})
        e.update(RANK=str(env.node_rank * nproc_per_node + lr), LOCAL_RANK=str(lr), WORLD_SIZE=str(world),
                 LOCAL_WORLD_SIZE=str(nproc_per_node), NODE_RANK=str(env.node_rank), NNODES=str(env.nnodes),
                 MASTER_ADDR=env.master_addr, MASTER_PORT=str(env.master_port),
                 CHATLEARN_HEARTBEAT_DIR=hb_dir, CLB200_ERROR_DIR=err_dir)
        if cpu:
            e["CHATLEARN_FORCE_CPU"] = "1"
        procs.append(subprocess.Popen(cmd, env=e, stdout=stdout, stderr=subprocess.STDOUT if stdout else None,
                                      start_new_session=True))
    failed = None
    try:
        while failed is None:
            alive = 0
            for lr, p in enumerate(procs):
                rc = p.poll()
                if rc is None:
                    alive += 1
                    hb = os.path.join(hb_dir, f"rank{env.node_rank * nproc_per_node + lr}")
                    if heartbeat_timeout_s > 0 and os.path.exists(hb) \
                            and time.time() - os.path.getmtime(hb) > heartbeat_timeout_s:
                        failed = f"local rank {lr}: heartbeat timeout"
                elif rc != 0:
                    failed = f"local rank {lr}: exit code {rc}"
            if failed is None and os.path.isdir(err_dir) and os.listdir(err_dir):
                name = sorted(os.listdir(err_dir))[0]
                with open(os.path.join(err_dir, name), encoding="utf-8") as f:
                    failed = f"{name[:-4]} reported {f.readline().strip()}"
            if failed is not None:
                try:
                    box.post_error(failed)
                except Exception:                            # head already gone: nothing to tell
                    pass
                break
            try:
                remote = box.error()
            except ConnectionError as e:
                remote = str(e)
            if remote is not None:
                failed = remote
                break
            if alive == 0:
                break
            time.sleep(poll_s)
        if failed is None:
            # this node is finished; node 0 serves the mailbox until every node is
            box.done()
            if env.node_rank == 0:
                deadline = time.time() + drain_timeout_s
                while not box.all_done() and time.time() < deadline:
                    if box.error() is not None:
                        failed = box.error()
                        break
                    time.sleep(poll_s)
    finally:
        if failed is not None:
            _stop(procs)
    if failed is not None:
        raise RankFailure(failed)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="per-node launcher of a multi-node job")
    ap.add_argument("--nproc-per-node", type=int, required=True)
    ap.add_argument("--cpu", action="store_true", help="CPU ranks (gloo)")
    ap.add_argument("--heartbeat-timeout", type=float, default=0.0)
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.cmd[1:] if a.cmd and a.cmd[0] == "--" else a.cmd
    assert cmd, "nothing to run"
    try:
        return launch_node(cmd, a.nproc_per_node, cpu=a.cpu, heartbeat_timeout_s=a.heartbeat_timeout)
    except RankFailure as e:
        print(f"[launcher] node {node_env().node_rank}: {e}", file=sys.stderr, flush=True)
        return 1


if __name__ == "__main__":
    sys.exit(main())
