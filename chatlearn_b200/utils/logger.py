"""Rank-aware logging.

Parity: chatlearn/utils/logger.py:24-98 (per-model logger with ip+rank prefix,
``log_rank_0``).  One process per GPU, so the prefix is ``[rank/world]``.
"""
import logging
import os
import sys

_FMT = "%(asctime)s %(levelname)s [%(rank)s] %(name)s: %(message)s"


class _RankFilter(logging.Filter):
    def filter(self, record):
        record.rank = f"{os.environ.get('RANK', '0')}/{os.environ.get('WORLD_SIZE', '1')}"
        return True


def setup_logger(name="chatlearn_b200", level=None):
    lg = logging.getLogger(name)
    if getattr(lg, "_cl_ready", False):
        return lg
    level = level or os.environ.get("CHATLEARN_LOG_LEVEL", "INFO")
    lg.setLevel(level)
    h = logging.StreamHandler(sys.stderr)
    h.setFormatter(logging.Formatter(_FMT, "%H:%M:%S"))
    h.addFilter(_RankFilter())
    lg.addHandler(h)
    lg.propagate = False
    lg._cl_ready = True
    return lg


logger = setup_logger()


def log_rank_0(msg, lg=None, level=logging.INFO):
    """Log only on global rank 0."""
    if int(os.environ.get("RANK", "0")) == 0:
        (lg or logger).log(level, msg)


def model_logger(model_name):
    return setup_logger(f"chatlearn_b200.{model_name}")
