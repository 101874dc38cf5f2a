"""Per-node launchers of a two-node job on one host (gloo): global ranks, error propagation from one
node to the other, and worker nodes leaving when the head node is gone."""
import os
import signal
import subprocess
import sys
import time

from chatlearn_b200.launcher.dlc_utils import get_free_ports, node_env

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, time
import torch, torch.distributed as dist
from chatlearn_b200.launcher.initialize import init_distributed
init_distributed()
r, w = dist.get_rank(), dist.get_world_size()
t = torch.tensor([float(r)])
dist.all_reduce(t)
print(f"RANK {r}/{w} node {os.environ['NODE_RANK']} sum {int(t.item())}", flush=True)
mode = os.environ.get("MODE", "ok")
if mode == "raise" and r == 3:
    raise RuntimeError("boom on rank 3")
if mode != "ok":
    time.sleep(120)          # the others wait (as in a collective) until their launcher stops them
'''


def _start(tmp_path, mode, port):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs, logs = [], []
    for node in (0, 1):
        env = dict(os.environ, NODE_RANK=str(node), NNODES="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   MODE=mode, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
            env.pop(k, None)
        log = open(tmp_path / f"node{node}.log", "w")
        logs.append(log)
        procs.append(subprocess.Popen([sys.executable, "-m", "chatlearn_b200.launcher.dlc_utils", "--nproc-per-node", "2",
                                       "--cpu", "--", sys.executable, str(script)], env=env, stdout=log,
                                      stderr=subprocess.STDOUT, start_new_session=True, cwd=ROOT))
    return procs, logs


def _wait(procs, timeout):
    deadline = time.time() + timeout
    try:
        return [p.wait(timeout=max(0.1, deadline - time.time())) for p in procs]
    finally:
        for p in procs:
            if p.poll() is None:
                os.killpg(p.pid, signal.SIGKILL)


def test_environment_parsing_and_ports():
    e = node_env({"WORLD_SIZE": "4", "RANK": "2", "LOCAL_MASTER_ADDR": "10.0.0.7", "CUSTOM_PORTS": "31001;31002,31003"})
    assert (e.node_rank, e.nnodes, e.master_addr, e.master_port) == (2, 4, "10.0.0.7", 31001)
    assert e.reserved_ports == [31001, 31002, 31003]
    import socket
    busy = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    busy.bind(("", 0))
    busy.listen(1)
    taken = busy.getsockname()[1]
    try:
        ports = get_free_ports(3, reserved=[taken, 31002], exclude=(31002,))   # one is in use, one is excluded
    finally:
        busy.close()
    assert len(set(ports)) == 3 and taken not in ports and 31002 not in ports


def test_two_nodes_run_to_completion(tmp_path):
    port = get_free_ports(2)[0]
    procs, _ = _start(tmp_path, "ok", port)
    assert _wait(procs, 120) == [0, 0]
    text = (tmp_path / "node0.log").read_text() + (tmp_path / "node1.log").read_text()
    assert all(f"RANK {r}/4 node {r // 2} sum 6" in text for r in range(4))


def test_failure_on_one_node_stops_the_other(tmp_path):
    port = get_free_ports(2)[0]
    procs, _ = _start(tmp_path, "raise", port)
    t0 = time.time()
    assert _wait(procs, 90) == [1, 1]
    assert time.time() - t0 < 80                                           # nobody sat out the 120 s sleep
    assert "exit code" in (tmp_path / "node0.log").read_text()            # node 0 learned of node 1's failure


def test_workers_leave_when_the_head_is_gone(tmp_path):
    port = get_free_ports(2)[0]
    procs, _ = _start(tmp_path, "hang", port)
    deadline = time.time() + 60
    while "sum 6" not in (tmp_path / "node1.log").read_text() and time.time() < deadline:
        time.sleep(0.5)
    os.killpg(procs[0].pid, signal.SIGKILL)                                # the head node's launcher and ranks vanish
    assert _wait(procs[1:], 90) == [1]
    assert "head node unreachable" in (tmp_path / "node1.log").read_text()
