"""`torch.profiler` traces (CPU + CUDA) and CUDA memory snapshots.

Two schedules: an explicit step range (``profile_step_start`` / ``profile_step_end``:
wait until two steps before the range, one warm-up step, one capture, no repeat) or the
frequency mode (every ``profile_freq`` steps capture ``profiler_active`` steps after
``profiler_warmup``).  ``profile_ranks`` restricts tracing to some ranks.  Online parse
writes Chrome/TensorBoard traces as they complete; offline mode exports one raw trace per
capture window for later parsing.

Memory snapshots record allocator history and dump a ``.pickle`` (viewable with
memory_viz) every ``profile_freq`` steps and on out-of-memory.

Parity: torchtitan_npu/tools/profiling.py:29-170, docs/feature_guides/metrics_and_debugging.md:75-109.
"""

from __future__ import annotations

import contextlib
import os
import pickle
import time

import torch

from titan_b200.utils.logging import logger

__all__ = ["is_profile_enabled", "compute_schedule", "maybe_enable_profiling", "maybe_enable_memory_snapshot", "nvtx_range"]


def is_profile_enabled(cfg, rank: int = 0) -> bool:
    if not cfg.enable_profiling:
        return False
    return cfg.profile_ranks == [-1] or rank in cfg.profile_ranks


def compute_schedule(cfg, global_step: int) -> dict | None:
    """→ ``dict(wait, warmup, active, repeat)`` or None when the window cannot be honoured."""
    if cfg.profile_step_start > 0:
        end = cfg.profile_step_end if cfg.profile_step_end > 0 else cfg.profile_step_start + cfg.profiler_active
        active = end - cfg.profile_step_start
        wait = cfg.profile_step_start - global_step - 2
        warmup = 1 if cfg.profile_step_start > global_step + 1 else 0
        repeat = 1
    else:
        warmup, active = cfg.profiler_warmup, cfg.profiler_active
        wait = cfg.profile_freq - (active + warmup)
        repeat = 0
    if wait < 0 or active <= 0:
        return None
    return {"wait": wait, "warmup": warmup, "active": active, "repeat": repeat}


@contextlib.contextmanager
def maybe_enable_profiling(cfg, *, global_step: int = 0, base_folder: str = "", rank: int = 0):
    if not is_profile_enabled(cfg, rank):
        yield None
        return
    sched = compute_schedule(cfg, global_step)
    if sched is None:
        logger.warning("profiling skipped: profile_step_start must exceed %d + 2, or profile_freq must be >= "
                       "warmup + active", global_step)
        yield None
        return
    trace_dir = os.path.join(base_folder, cfg.save_traces_folder)
    os.makedirs(trace_dir, exist_ok=True)
    logger.info("profiling rank %d with schedule %s → %s", rank, sched, trace_dir)

    def offline_handler(prof):
        path = os.path.join(trace_dir, f"rank{rank}_step{prof.step_num}_raw.json")
        prof.export_chrome_trace(path)
        logger.info("raw profiler trace saved at %s", path)

    if cfg.enable_online_parse:
        handler = torch.profiler.tensorboard_trace_handler(trace_dir, worker_name=f"rank{rank}")
    else:
        handler = offline_handler
    activities = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        activities.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(
        activities=activities,
        schedule=torch.profiler.schedule(**sched),
        on_trace_ready=handler,
        record_shapes=cfg.profile_record_shapes,
        profile_memory=cfg.profile_with_memory,
        with_stack=cfg.profile_with_stack,
    ) as prof:
        prof.step_num = global_step
        yield prof


class _MemorySnapshot:
    MAX_ENTRIES = 100000

    def __init__(self, folder: str, freq: int, rank: int, global_step: int):
        self.folder, self.freq, self.rank, self.step_num = folder, freq, rank, global_step
        torch.cuda.memory._record_memory_history(max_entries=self.MAX_ENTRIES)

    def step(self, exit_ctx: bool = False) -> None:
        self.step_num += 1
        if not exit_ctx and self.step_num % self.freq != 0:
            return
        tag = f"iteration_{self.step_num}" + ("_exit" if exit_ctx else "")
        out = os.path.join(self.folder, tag)
        os.makedirs(out, exist_ok=True)
        begin = time.monotonic()
        with open(os.path.join(out, f"rank{self.rank}_memory_snapshot.pickle"), "wb") as f:
            pickle.dump(torch.cuda.memory._snapshot(), f)
        logger.info("memory snapshot dumped in %.2f s", time.monotonic() - begin)


@contextlib.contextmanager
def maybe_enable_memory_snapshot(cfg, *, global_step: int = 0, base_folder: str = "", rank: int = 0):
    if not cfg.enable_memory_snapshot or not torch.cuda.is_available():
        yield None
        return
    folder = os.path.join(base_folder, cfg.save_memory_snapshot_folder)
    os.makedirs(folder, exist_ok=True)
    snap = _MemorySnapshot(folder, cfg.profile_freq, rank, global_step)
    try:
        yield snap
    except torch.OutOfMemoryError:
        snap.step(exit_ctx=True)
        raise
    finally:
        torch.cuda.memory._record_memory_history(enabled=None)


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = True):
    """NVTX range around a fused kernel or trainer phase (no-op without CUDA)."""
    if enabled and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield
