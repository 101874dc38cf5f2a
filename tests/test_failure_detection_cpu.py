"""Failure detection by the job supervisor, with failures made on the host: a rank that
raises, a rank that exits, a rank that stops beating while its peers wait in a collective."""
import sys
import time


from chatlearn_b200.launcher.local import RankFailure, launch_local

PRE = r'''
import os, sys, time, datetime
import torch, torch.distributed as dist
from chatlearn_b200.launcher.local import Heartbeat
hb = Heartbeat(interval_s=0.2)
rank = int(os.environ["RANK"])
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
dist.barrier()
'''


def _run(body, **kw):
    t0 = time.time()
    try:
        launch_local([sys.executable, "-c", PRE + body], nproc=2, cpu=True, poll_s=0.1, **kw)
        return None, time.time() - t0
    except RankFailure as e:
        return str(e), time.time() - t0


def test_healthy_job_returns_zero():
    err, _ = _run("dist.barrier()\n")
    assert err is None


def test_rank_that_raises_ends_the_job():
    # rank 1 dies between steps; rank 0 would wait 120 s in the next collective without the supervisor
    err, dt = _run("if rank == 1:\n    raise RuntimeError('boom')\ndist.barrier()\n")
    assert err is not None and "rank 1" in err and dt < 60


def test_reported_exception_is_named():
    body = ("from chatlearn_b200.runtime.decorator import monitor_error\n"
            "class R:\n    name = 'policy'\n    @monitor_error()\n    def forward_step(self):\n        raise ValueError('bad batch')\n"
            "if rank == 0:\n    try:\n        R().forward_step()\n    except ValueError:\n        time.sleep(30)\n"
            "dist.barrier()\n")
    err, dt = _run(body)
    assert err is not None and "rank 0" in err and "policy.forward_step" in err and dt < 25


def test_wedged_rank_is_found_by_its_heartbeat():
    # rank 1 stops beating and never joins; nothing exits on its own
    body = "if rank == 1:\n    hb.pause()\n    time.sleep(60)\nelse:\n    dist.barrier()\n"
    err, dt = _run(body, heartbeat_timeout_s=2.0)
    assert err is not None and "heartbeat" in err and "rank 1" in err and dt < 40


def test_silent_exit_code():
    err, _ = _run("if rank == 0:\n    os._exit(3)\ndist.barrier()\n")
    assert err is not None and "exit code 3" in err


def test_log_lines_of_all_nodes_reach_node_zero(tmp_path):
    """Two "nodes" tail their rank logs and publish through a key-value store; node 0 shows both, with node and rank
    prefixes, keeps the error-like lines, and ordinary lines beyond the rate limit stay local."""
    from datetime import timedelta

    from torch.distributed import TCPStore

    from chatlearn_b200.utils.log_monitor import LogMonitor, StoreLogCollector, StoreLogPublisher
    from chatlearn_b200.utils.utils import get_free_port
    port = get_free_port()
    server = TCPStore("127.0.0.1", port, None, True, timeout=timedelta(seconds=20), wait_for_workers=False)
    client = TCPStore("127.0.0.1", port, None, False, timeout=timedelta(seconds=20), wait_for_workers=False)
    dirs = [tmp_path / "n0", tmp_path / "n1"]
    for d in dirs:
        d.mkdir()
    (dirs[0] / "rank0.log").write_text("step 1 ok\n")
    (dirs[1] / "rank5.log").write_text("step 1 ok\nRuntimeError: CUDA error: an illegal memory access\n" + "noise\n" * 100)
    mons = [LogMonitor(str(dirs[0]), sink=StoreLogPublisher(server, 0, max_lines_per_s=5)),
            LogMonitor(str(dirs[1]), sink=StoreLogPublisher(client, 1, max_lines_per_s=5))]
    seen = []
    col = StoreLogCollector(server, 2, sink=seen.append)
    for m in mons:
        m.poll()
    col.poll()
    assert "(node0:rank0) step 1 ok" in seen and "(node1:rank5) step 1 ok" in seen
    assert any("illegal memory access" in e and e.startswith("(node1:rank5)") for e in col.errors)
    assert sum("noise" in s for s in seen) <= 5
