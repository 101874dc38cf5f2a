"""Failure detection by the job supervisor, with failures made on the host: a rank that
raises, a rank that exits, a rank that stops beating while its peers wait in a collective."""
import sys
import time

import pytest

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
