"""Context-parallel strategy registry.

A strategy is a ``(detector, applier)`` pair: the first detector that accepts an attention module
decides how CP hooks are attached; a module nobody accepts raises `NotImplementedError`.  Mask
handlers ``(masks, cp_mesh) -> per-rank masks | None`` adapt custom mask / metadata types to the
sequence shard of a rank.

Parity: torchtitan_npu/distributed/context_parallel/registry.py:21-98.
"""

from __future__ import annotations

from collections.abc import Callable

import torch.nn as nn
from torch.distributed.device_mesh import DeviceMesh

__all__ = ["register_cp_strategy", "apply_cp_to_attention_module", "register_cp_mask_handler", "adjust_cp_mask",
           "registered_strategies"]

_STRATEGIES: list[tuple[str, Callable, Callable]] = []
_MASK_HANDLERS: list[Callable] = []


def register_cp_strategy(name: str, detector: Callable[[nn.Module], bool],
                         applier: Callable[[nn.Module, DeviceMesh], nn.Module], *, first: bool = False) -> None:
    entry = (name, detector, applier)
    for i, (n, _, _) in enumerate(_STRATEGIES):
        if n == name:
            _STRATEGIES[i] = entry
            return
    if first:
        _STRATEGIES.insert(0, entry)
    else:
        _STRATEGIES.append(entry)


def registered_strategies() -> list[str]:
    return [n for n, _, _ in _STRATEGIES]


def apply_cp_to_attention_module(modules: list[nn.Module], cp_mesh: DeviceMesh) -> list[str]:
    """Attach CP hooks to each module; returns the strategy name chosen per module."""
    chosen = []
    for mod in modules:
        for name, detect, apply in _STRATEGIES:
            if detect(mod):
                apply(mod, cp_mesh)
                chosen.append(name)
                break
        else:
            raise NotImplementedError(
                f"no context-parallel strategy accepts {type(mod).__name__}; registered: {registered_strategies()}")
    return chosen


def register_cp_mask_handler(handler: Callable) -> None:
    if handler not in _MASK_HANDLERS:
        _MASK_HANDLERS.append(handler)


def adjust_cp_mask(masks, cp_mesh: DeviceMesh):
    for h in _MASK_HANDLERS:
        out = h(masks, cp_mesh)
        if out is not None:
            return out
    return masks
