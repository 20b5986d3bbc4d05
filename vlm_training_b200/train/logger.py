"""Rank-aware console logging (reference: train/logger.py:1-50).

Rank 0 logs at INFO to stdout; every other rank logs errors only and has
Python warnings silenced, so an 8-rank job prints one copy of each line.
"""
from __future__ import annotations

import logging
import os
import sys
import warnings


class Color:
    black = "\033[30m"
    red = "\033[31m"
    green = "\033[32m"
    yellow = "\033[33m"
    blue = "\033[34m"
    magenta = "\033[35m"
    cyan = "\033[36m"
    white = "\033[37m"
    reset = "\033[0m"
    bold = "\033[1m"


class NoColor:
    black = red = green = yellow = blue = magenta = cyan = white = reset = bold = ""


logger = logging.getLogger("vlm_training_b200")


def init_logger(rank: int | None = None) -> logging.Logger:
    if rank is None:
        rank = int(os.environ.get("RANK", "0"))
    logger.handlers.clear()
    handler = logging.StreamHandler(sys.stdout)
    handler.setFormatter(logging.Formatter(f"[rank {rank}] %(asctime)s %(levelname)s %(message)s", "%H:%M:%S"))
    logger.addHandler(handler)
    logger.propagate = False
    if rank == 0:
        logger.setLevel(logging.INFO)
    else:
        logger.setLevel(logging.ERROR)
        warnings.filterwarnings("ignore")
    return logger


def colors():
    return Color if sys.stdout.isatty() else NoColor
