"""Process bootstrap: global args and the job-wide process group.

Parity: chatlearn/launcher/initialize.py:92-111 (``chatlearn.init(args)``).  The
reference starts / joins a Ray cluster; here ``init`` joins the
``torch.distributed`` job described by ``RANK / WORLD_SIZE / MASTER_ADDR /
MASTER_PORT`` (torchrun, or this package's local launcher): NCCL when the process
has a GPU, gloo otherwise, plus a gloo side group for host-side object exchange
and heartbeats.
"""
import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist

from chatlearn_b200.utils import global_vars
from chatlearn_b200.utils.logger import logger

_CPU_GROUP = None


def cpu_group():
    return _CPU_GROUP


def init_distributed(timeout_s: float = 1800.0, backend: Optional[str] = None):
    global _CPU_GROUP
    if dist.is_initialized():
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1 and "MASTER_ADDR" not in os.environ:
        return
    rank = int(os.environ.get("RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    use_cuda = torch.cuda.is_available() and os.environ.get("CHATLEARN_FORCE_CPU", "0") != "1"
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    backend = backend or ("cpu:gloo,cuda:nccl" if use_cuda else "gloo")
    kw = {}
    if use_cuda:
        kw["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group(backend=backend, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s), **kw)
    logger.info(f"joined job: rank {rank}/{world} backend {backend}")


def init(args=None, config_file: Optional[str] = None, overrides=None):
    """Set the global configuration and join the distributed job.

    ``args``: a config object with ``runtime_args`` and ``models`` (e.g. ``GrpoConfig``).
    With ``args=None`` a YAML file (``config_file`` or ``-c`` on the command line) is
    parsed with the legacy loader."""
    if args is None:
        from chatlearn_b200.utils.arguments import parse_args
        args = parse_args(config_file, overrides)
    global_vars.set_global_variables(args)
    ra = args.runtime_args
    init_distributed(timeout_s=float(getattr(ra, "distributed_timeout_s", 1800.0)))
    return args


def shutdown(grace_s: float = 20.0):
    """End a distributed job: synchronise, release CUDA graphs and cached blocks, then
    destroy the process group.  NCCL's teardown can block when captured graphs that
    contain its kernels are still alive, so a watchdog thread ends the process once
    ``grace_s`` has passed; by then every result has been flushed by the caller."""
    import gc
    import os
    import sys
    import threading
    if not dist.is_initialized():
        return
    sys.stdout.flush()
    sys.stderr.flush()
    t = threading.Timer(grace_s, lambda: os._exit(0))
    t.daemon = True
    t.start()
    try:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        gc.collect()
        dist.barrier()
        dist.destroy_process_group()
    finally:
        t.cancel()
