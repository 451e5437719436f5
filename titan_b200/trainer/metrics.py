"""Per-step metrics: loss, grad-norm, tokens/s, TFLOP/s, MFU, step time, memory.

Throughput is ``tokens / (Δt · non_data_parallel_size)`` (tokens per second per
data-parallel replica slice, i.e. per GPU); ``mfu = 100 · flops_per_token · tps / peak``
and is omitted when a low-precision converter is active (the bf16 peak would be the
wrong denominator).  Δt is device time from CUDA events (max over ranks) when
``metrics.device_timed`` is on and CUDA is present, else host `perf_counter`.

Parity: torchtitan_npu/patches/tools/metrics.py:42-122 (console line with
``elapsed_time_per_step``, quantised-run MFU rule, peak table).
"""

from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Any

import torch

from titan_b200.utils.device import get_peak_flops
from titan_b200.utils.logging import logger

__all__ = ["MetricsProcessor", "DeviceMemoryMonitor", "StepTimer"]


@dataclass
class _MemStats:
    max_active_gib: float
    max_active_pct: float
    max_reserved_gib: float
    max_reserved_pct: float
    num_alloc_retries: int
    num_ooms: int


class DeviceMemoryMonitor:
    def __init__(self):
        self.cuda = torch.cuda.is_available()
        self.capacity = torch.cuda.get_device_properties(0).total_memory if self.cuda else 1
        self.device_name = torch.cuda.get_device_name(0) if self.cuda else "cpu"

    def get_peak_stats(self) -> _MemStats:
        if not self.cuda:
            return _MemStats(0, 0, 0, 0, 0, 0)
        info = torch.cuda.memory_stats()
        act = info.get("active_bytes.all.peak", 0)
        res = info.get("reserved_bytes.all.peak", 0)
        gib = 1024 ** 3
        return _MemStats(act / gib, 100 * act / self.capacity, res / gib, 100 * res / self.capacity,
                         info.get("num_alloc_retries", 0), info.get("num_ooms", 0))

    def reset_peak_stats(self) -> None:
        if self.cuda:
            torch.cuda.reset_peak_memory_stats()


class StepTimer:
    """Device-side interval timer (CUDA events) with a host-clock fallback."""

    def __init__(self, device_timed: bool):
        self.use_events = device_timed and torch.cuda.is_available()
        self._start_evt = None
        self._t0 = time.perf_counter()

    def start(self) -> None:
        if self.use_events:
            self._start_evt = torch.cuda.Event(enable_timing=True)
            self._start_evt.record()
        self._t0 = time.perf_counter()

    def stop(self) -> float:
        """Seconds since `start()`."""
        if self.use_events and self._start_evt is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            end.synchronize()
            return self._start_evt.elapsed_time(end) / 1e3
        return time.perf_counter() - self._t0


class MetricsProcessor:
    def __init__(self, config, *, parallel_dims, dump_folder: str = "", quantized: bool = False, rank: int = 0):
        self.config = config
        self.parallel_dims = parallel_dims
        self.quantized = quantized
        self.rank = rank
        self.monitor = DeviceMemoryMonitor()
        self.peak_flops = get_peak_flops(self.monitor.device_name)
        self.num_flops_per_token = 0
        self.ntokens_since_last_log = 0
        self.data_loading_times: list[float] = []
        self.timer = StepTimer(config.device_timed)
        self.timer.start()
        self.steps_since_last_log = 0
        self.history: list[dict[str, Any]] = []
        self.writer = None
        if config.enable_tensorboard and (rank == 0 or config.save_for_all_ranks):
            from torch.utils.tensorboard import SummaryWriter

            self.writer = SummaryWriter(os.path.join(dump_folder, config.save_tb_folder), max_queue=1000)

    def should_log(self, step: int) -> bool:
        return step == 1 or step % self.config.log_freq == 0

    def log(self, step: int, global_avg_loss: float, global_max_loss: float, grad_norm: float,
            extra_metrics: dict[str, Any] | None = None, loss_mesh=None) -> dict[str, Any]:
        elapsed = self.timer.stop()
        if loss_mesh is not None:
            from titan_b200.parallel.utils import dist_max

            elapsed = dist_max(elapsed, loss_mesh)
        nd = self.parallel_dims.non_data_parallel_size
        tps = self.ntokens_since_last_log / max(elapsed * nd, 1e-12)
        tflops = self.num_flops_per_token * tps / 1e12
        mfu = None if self.quantized else 100 * self.num_flops_per_token * tps / self.peak_flops
        steps = max(self.steps_since_last_log, 1)
        per_step = elapsed / steps
        data_t = sum(self.data_loading_times) / max(len(self.data_loading_times), 1)
        mem = self.monitor.get_peak_stats()
        metrics = {
            "loss_metrics/global_avg_loss": global_avg_loss,
            "loss_metrics/global_max_loss": global_max_loss,
            "grad_norm": grad_norm,
            "throughput(tps)": tps,
            "tflops": tflops,
            "time_metrics/end_to_end(s)": per_step,
            "time_metrics/data_loading(s)": data_t,
            "time_metrics/data_loading(%)": 100 * data_t / max(per_step, 1e-12),
            "memory/max_active(GiB)": mem.max_active_gib,
            "memory/max_active(%)": mem.max_active_pct,
            "memory/max_reserved(GiB)": mem.max_reserved_gib,
            "memory/max_reserved(%)": mem.max_reserved_pct,
            "memory/num_alloc_retries": mem.num_alloc_retries,
            "memory/num_ooms": mem.num_ooms,
        }
        if mfu is not None:
            metrics["mfu(%)"] = mfu
        if extra_metrics:
            metrics.update(extra_metrics)
        if self.writer is not None:
            for k, v in metrics.items():
                if isinstance(v, (int, float)):
                    self.writer.add_scalar(k, v, step)
        mfu_txt = "  mfu: n/a (quantized)" if mfu is None else f"  mfu: {mfu:.2f}%"
        logger.info(
            "step: %2d  loss: %7.4f  grad_norm: %7.4f  memory: %5.2fGiB(%.2f%%)  tps: %s  tflops: %.2f%s  "
            "elapsed_time_per_step: %.4fs",
            step, global_avg_loss, grad_norm, mem.max_reserved_gib, mem.max_reserved_pct,
            f"{round(tps):,}", tflops, mfu_txt, per_step,
        )
        self.history.append({"step": step, **metrics})
        self.ntokens_since_last_log = 0
        self.steps_since_last_log = 0
        self.data_loading_times.clear()
        self.monitor.reset_peak_stats()
        self.timer.start()
        return metrics

    def close(self) -> None:
        if self.writer is not None:
            self.writer.close()
