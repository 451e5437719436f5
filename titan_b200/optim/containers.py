"""Optimizer and LR-scheduler containers + the builder that dispatches on the config.

`build_optimizers` picks one of: standard (torch AdamW/Adam or the sm_100a
multi-tensor fused AdamW), Swap (state in pinned host memory), Virtual (state in
host-mapped memory), Muon hybrid, or Swap-Muon.  Virtual and Swap are mutually
exclusive.

State dicts are flattened per parameter FQN (``state.<fqn>.exp_avg`` …,
``param_groups.<fqn>.lr`` …) so DCP can reshard optimizer state across
different parallel layouts.

Parity: torchtitan_npu/patches/optimizer/optimizer_selector.py:34-210
(dispatch rules), upstream `OptimizersContainer` / `LRSchedulersContainer`
semantics, warmup-stable-decay schedule (muon_optimizer.py:1496-1559).
"""

from __future__ import annotations

import functools
import math
from typing import Any

import torch
import torch.nn as nn
from torch.distributed.checkpoint.state_dict import (
    StateDictOptions,
    get_optimizer_state_dict,
    set_optimizer_state_dict,
)
from torch.distributed.checkpoint.stateful import Stateful
from torch.optim import Optimizer
from torch.optim.lr_scheduler import LambdaLR

__all__ = [
    "OptimizersContainer",
    "LRSchedulersContainer",
    "build_optimizers",
    "build_lr_schedulers",
    "linear_warmup_stable_decay",
]


def _adam_kwargs(cfg) -> dict[str, Any]:
    kw = dict(lr=cfg.lr, betas=(cfg.beta1, cfg.beta2), eps=cfg.eps, weight_decay=cfg.weight_decay)
    impl = cfg.implementation
    if impl == "fused":
        kw["fused"] = True
    elif impl == "foreach":
        kw["foreach"] = True
    elif impl == "for-loop":
        kw["foreach"] = False
    return kw


class OptimizersContainer(Optimizer, Stateful):
    """One optimizer per model part (pipeline stages), stepped together."""

    def __init__(self, model_parts: list[nn.Module], optimizer_cls: type[Optimizer], optimizer_kwargs: dict[str, Any]):
        self.model_parts = model_parts
        self.optimizers: list[Optimizer] = []
        all_params = []
        for part in model_parts:
            params = [p for p in part.parameters() if p.requires_grad]
            self.optimizers.append(optimizer_cls(params, **optimizer_kwargs))
            all_params.extend(params)
        # base-class init so hooks (step pre/post hooks) can be registered on the container
        Optimizer.__init__(self, all_params, optimizer_kwargs)

    def __iter__(self):
        return iter(self.optimizers)

    def __len__(self):
        return len(self.optimizers)

    def step(self, *args, **kwargs) -> None:
        for opt in self.optimizers:
            opt.step(*args, **kwargs)
    def zero_grad(self, *args, **kwargs) -> None:
        for opt in self.optimizers:
            opt.zero_grad(*args, **kwargs)

    def state_dict(self) -> dict[str, Any]:
        opts = StateDictOptions(flatten_optimizer_state_dict=True)
        out: dict[str, Any] = {}
        for part, opt in zip(self.model_parts, self.optimizers):
            out.update(get_optimizer_state_dict(part, opt, options=opts))
        return out

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        opts = StateDictOptions(flatten_optimizer_state_dict=True)
        for part, opt in zip(self.model_parts, self.optimizers):
            set_optimizer_state_dict(part, opt, optim_state_dict=state_dict, options=opts)

    def init_cache_state_dict(self) -> None:
        """Optimizers whose state is not on the device cache it here before an async save."""


def linear_warmup_stable_decay(step: int, *, warmup_steps: int, stable_steps: int, decay_steps: int,
                               decay_type: str, min_lr_factor: float) -> float:
    """LR multiplier: linear warmup → flat → linear / sqrt / cosine decay to `min_lr_factor`."""
    if step < warmup_steps:
        return float(step + 1) / float(warmup_steps + 1)
    if step < warmup_steps + stable_steps:
        return 1.0
    if decay_steps <= 0:
        return 1.0
    progress = min(1.0, float(step + 1 - warmup_steps - stable_steps) / float(decay_steps))
    if decay_type == "linear":
        f = 1 - progress
    elif decay_type == "sqrt":
        f = 1 - math.sqrt(progress)
    elif decay_type == "cosine":
        f = 0.5 * (1.0 + math.cos(math.pi * progress))
    else:
        raise ValueError(f"unknown decay_type {decay_type!r}")
    return min_lr_factor + (1 - min_lr_factor) * f


class LRSchedulersContainer(Stateful):
    def __init__(self, optimizers, lr_lambda):
        self.schedulers = [LambdaLR(opt, lr_lambda) for opt in optimizers]

    def __iter__(self):
        return iter(self.schedulers)

    def step(self) -> None:
        for s in self.schedulers:
            s.step()

    def state_dict(self) -> dict[str, Any]:
        # all schedulers advance in lock-step, so one state restores them all
        return self.schedulers[0].state_dict() if self.schedulers else {}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        import copy

        for s in self.schedulers:
            s.load_state_dict(copy.deepcopy(state_dict))


def build_lr_schedulers(optimizers, lr_cfg, training_steps: int):
    warmup = int(lr_cfg.warmup_steps)
    if warmup > training_steps:
        warmup = training_steps
    if lr_cfg.decay_ratio is not None:
        decay = round(training_steps * lr_cfg.decay_ratio)
        if warmup + decay > training_steps:
            decay = training_steps - warmup
    else:
        decay = training_steps - warmup
    stable = training_steps + 1 - warmup - decay
    fn = functools.partial(linear_warmup_stable_decay, warmup_steps=warmup, stable_steps=stable, decay_steps=decay,
                           decay_type=lr_cfg.decay_type, min_lr_factor=lr_cfg.min_lr_factor)
    inner = getattr(optimizers, "lr_scheduler_targets", None)
    targets = inner() if callable(inner) else list(optimizers)
    return LRSchedulersContainer(targets, fn)


def build_optimizers(model_parts: list[nn.Module], opt_cfg, parallel_dims=None, ft_manager=None, *,
                     cuda_graph: bool = False):
    """Dispatch on the optimizer config (see module docstring).  ``cuda_graph`` (`--compile.cuda_graphs`) records the
    step of the fused AdamW as a CUDA graph."""
    if opt_cfg.virtual_optimizer and opt_cfg.swap_optimizer:
        raise ValueError("virtual_optimizer and swap_optimizer cannot be enabled together")
    name = opt_cfg.name
    if name == "Muon":
        from titan_b200.optim.muon import build_muon_optimizers

        return build_muon_optimizers(model_parts, opt_cfg, parallel_dims, swap=opt_cfg.swap_optimizer)
    if name not in ("AdamW", "Adam"):
        raise NotImplementedError(f"optimizer {name!r} is not supported (AdamW, Adam, Muon)")
    if opt_cfg.virtual_optimizer:
        from titan_b200.optim.virtual_optimizer import VirtualOptimizersContainer

        return VirtualOptimizersContainer(model_parts, opt_cfg, parallel_dims)
    if opt_cfg.swap_optimizer:
        from titan_b200.optim.swap_optimizer import SwapOptimizersContainer

        return SwapOptimizersContainer(model_parts, opt_cfg)
    if opt_cfg.implementation == "b200_fused":
        from titan_b200.optim.fused_adamw import FusedAdamW

        kw = dict(lr=opt_cfg.lr, betas=(opt_cfg.beta1, opt_cfg.beta2), eps=opt_cfg.eps,
                  weight_decay=opt_cfg.weight_decay, decoupled=(name == "AdamW"), cuda_graph=cuda_graph)
        return OptimizersContainer(model_parts, FusedAdamW, kw)
    cls = torch.optim.AdamW if name == "AdamW" else torch.optim.Adam
    return OptimizersContainer(model_parts, cls, _adam_kwargs(opt_cfg))
