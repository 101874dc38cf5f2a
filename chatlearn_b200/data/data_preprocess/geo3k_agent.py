"""Geometry3K for the answer-checking agent (chatlearn/data/data_preprocess/geo3k_agent.py)."""
from .common import run_converter
from .geo3k import convert as _convert


def convert(ex, split, idx):
    return _convert(ex, split, idx, agent=True)


if __name__ == "__main__":
    run_converter(__doc__, "~/data/geo3k", convert, suffix="_agent")
