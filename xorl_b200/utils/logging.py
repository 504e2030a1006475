"""Rank-aware logging helpers (``info_rank0``, ``warning_once``), cf. src/xorl/utils/logging.py."""
from __future__ import annotations

import logging
import os
import sys
from functools import lru_cache

_FMT = "[%(levelname)s][%(name)s:%(lineno)d] %(asctime)s >> %(message)s"


def get_logger(name: str = "xorl_b200") -> logging.Logger:
    lg = logging.getLogger(name)
    if not lg.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter(_FMT, "%m/%d/%Y %H:%M:%S"))
        lg.addHandler(h)
        lg.setLevel(os.environ.get("XORL_LOG_LEVEL", "INFO"))
        lg.propagate = False
    return lg


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


def info_rank0(msg: str, *a) -> None:
    if _rank() == 0:
        get_logger().info(msg, *a)


def warning_rank0(msg: str, *a) -> None:
    if _rank() == 0:
        get_logger().warning(msg, *a)


@lru_cache(maxsize=None)
def warning_once(msg: str) -> None:
    get_logger().warning(msg)
