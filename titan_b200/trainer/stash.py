"""Process-wide view of the active trainer config and parallel dims.

Narrow builders (loss, dataloader, optimizer, model configs) sometimes need trainer
fields they are not handed (MTP count, meshes).  The trainer publishes them here once
at construction; `clear()` runs at `Trainer.close()`.  Hooks registered by converters or
models (`post_dataloading`, `metrics`) are also kept here.

Parity: torchtitan_npu/patches/torchtitan/_trainer_config_stash.py:38-85.
"""

from __future__ import annotations

from collections.abc import Callable

__all__ = [
    "set_trainer_config", "get_trainer_config", "set_active_parallel_dims", "get_active_parallel_dims",
    "register_post_dataloading_hook", "post_dataloading_hooks", "register_metrics_hook", "metrics_hooks", "clear",
]

_STATE: dict = {"config": None, "parallel_dims": None, "post_dl": [], "metrics": []}


def set_trainer_config(cfg) -> None:
    _STATE["config"] = cfg


def get_trainer_config():
    return _STATE["config"]


def set_active_parallel_dims(pd) -> None:
    _STATE["parallel_dims"] = pd


def get_active_parallel_dims():
    return _STATE["parallel_dims"]


def register_post_dataloading_hook(fn: Callable) -> None:
    """``fn(trainer, inputs, labels, extra_inputs, extra_kwargs) -> same 4-tuple``."""
    if fn not in _STATE["post_dl"]:
        _STATE["post_dl"].append(fn)


def post_dataloading_hooks() -> list[Callable]:
    return list(_STATE["post_dl"])


def register_metrics_hook(fn: Callable) -> None:
    """``fn(trainer) -> dict`` of extra metrics, called on log steps only."""
    if fn not in _STATE["metrics"]:
        _STATE["metrics"].append(fn)


def metrics_hooks() -> list[Callable]:
    return list(_STATE["metrics"])


def clear() -> None:
    _STATE.update(config=None, parallel_dims=None, post_dl=[], metrics=[])
