"""Scheduled garbage collection: Python's automatic GC is disabled and a generation-1
collection runs every `gc_freq` steps, so all ranks pause at the same step instead of
stalling collectives at random.

Parity: the upstream `GarbageCollection.run` the reference wraps (train.py:108-133; its
extra "empty the device cache at step 1" lives in `Trainer.train`).
"""

from __future__ import annotations

import gc
import time

from titan_b200.utils.logging import logger

__all__ = ["GarbageCollection"]


class GarbageCollection:
    def __init__(self, gc_freq: int = 50, debug: bool = False):
        if gc_freq <= 0:
            raise ValueError("gc_freq must be positive")
        self.gc_freq = gc_freq
        self.debug = debug
        gc.disable()
        self.collect("initial GC collection")
        if debug:
            gc.set_debug(gc.DEBUG_STATS)

    def run(self, step_count: int) -> None:
        if self.debug:
            self.collect("debug GC collection", generation=2)
        elif step_count > 1 and step_count % self.gc_freq == 0:
            self.collect("periodic GC collection")

    @staticmethod
    def collect(reason: str, generation: int = 1) -> None:
        begin = time.monotonic()
        gc.collect(generation)
        logger.debug("[GC] %s took %.2f s", reason, time.monotonic() - begin)
