"""Package logger; rank filtering follows ``LOG_RANK`` (comma-separated ranks, default all)."""

from __future__ import annotations

import logging
import os

__all__ = ["logger", "init_logger"]

logger = logging.getLogger("titan_b200")


def init_logger(level: int = logging.INFO) -> None:
    if logger.handlers:
        return
    rank = int(os.environ.get("RANK", "0"))
    wanted = os.environ.get("LOG_RANK")
    handler = logging.StreamHandler()
    handler.setFormatter(logging.Formatter(f"[titan_b200 r{rank}] %(asctime)s %(levelname)s %(message)s", "%H:%M:%S"))
    logger.addHandler(handler)
    logger.propagate = False
    if wanted is not None and str(rank) not in [r.strip() for r in wanted.split(",")]:
        logger.setLevel(logging.ERROR)
    else:
        logger.setLevel(level)
