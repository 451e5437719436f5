"""Model-converter protocol and registry.

A converter is an opt-in, per-recipe rewrite applied after the model is built
(on the meta device) and before it is parallelised.  One registered name may
bundle three parts:

* a *model converter*  – swaps modules / functions for fused sm_100a versions;
* a *plan updater*     – rewrites tensor/expert-parallel plans (e.g. the NCCL
  expert-parallel style → the fused peer-memory style);
* a *state-dict updater* – keeps checkpoints in the canonical layout although
  the converted module stores parameters differently (e.g. fused ``w13``).

Parity: `ModelCustomConfig(model_converter, parallelize_plan_updater,
state_dict_updater)` and `register_model_converter / get_model_converter_config
/ has_npu_converter` (torchtitan_npu/converters/model_custom_interface.py:14-60,
converters/registry.py:12-39, converters/framework/*.py).  The reference
monkey-patches `parallelize_module` and subclasses adapters at run time; here
the trainer and the plan helper consult the registry directly.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Any

import torch.nn as nn

__all__ = [
    "ModelConverter",
    "PlanUpdater",
    "StateDictUpdater",
    "ConverterSpec",
    "ConverterConfig",
    "register_model_converter",
    "get_model_converter_config",
    "has_converter",
    "ModelConvertersContainer",
    "active_plan_updaters",
    "active_state_dict_updaters",
    "reset_active_converters",
    "converter_names",
]


class ModelConverter(ABC):
    def __init__(self, model_spec=None, trainer_config=None):
        self.model_spec = model_spec
        self.trainer_config = trainer_config
        self.model_name = getattr(model_spec, "name", None)

    @abstractmethod
    def convert(self, model: nn.Module) -> None: ...

    def post_optimizer_hook(self, model_parts) -> None:
        """Called after every optimizer step (low-precision converters refresh scales here)."""


class PlanUpdater(ABC):
    @classmethod
    @abstractmethod
    def update(cls, plan): ...


class StateDictUpdater(ABC):
    @classmethod
    @abstractmethod
    def to_hf(cls, state_dict: dict[str, Any]) -> dict[str, Any]: ...

    @classmethod
    @abstractmethod
    def from_hf(cls, state_dict: dict[str, Any]) -> dict[str, Any]: ...


@dataclass
class ConverterSpec:
    name: str = "default"
    model_converter: type[ModelConverter] | None = None
    plan_updater: type[PlanUpdater] | None = None
    state_dict_updater: type[StateDictUpdater] | None = None
    aliases: tuple[str, ...] = ()


@dataclass
class ConverterConfig:
    """What a recipe lists in ``model_converters.converters``."""

    name: str
    options: dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> dict:
        return {"name": self.name, **self.options}


_REGISTRY: dict[str, ConverterSpec] = {}
_ALIASES: dict[str, str] = {}
_ACTIVE_PLAN_UPDATERS: list[type[PlanUpdater]] = []
_ACTIVE_SD_UPDATERS: list[type[StateDictUpdater]] = []


def register_model_converter(name: str, *aliases: str):
    """Decorator: ``@register_model_converter("b200_rms_norm", "npu_rms_norm")`` on a `ConverterSpec`."""

    def deco(spec: ConverterSpec) -> ConverterSpec:
        spec.name = name
        spec.aliases = tuple(aliases)
        _REGISTRY[name] = spec
        for a in aliases:
            _ALIASES[a] = name
        return spec

    return deco


def _canonical(name: str) -> str:
    return _ALIASES.get(name, name)


def _ensure_discovered() -> None:
    import titan_b200.converters  # noqa: F401  (imports every converter module)


def converter_names() -> list[str]:
    _ensure_discovered()
    return sorted(_REGISTRY)


def get_model_converter_config(name: str, **options) -> ConverterConfig:
    _ensure_discovered()
    canon = _canonical(name)
    if canon not in _REGISTRY:
        raise KeyError(f"unknown model converter {name!r}; registered: {sorted(_REGISTRY)}")
    return ConverterConfig(name=canon, options=dict(options))


def _name_of(entry) -> str | None:
    if isinstance(entry, str):
        return _canonical(entry)
    n = getattr(entry, "name", None)
    return _canonical(n) if isinstance(n, str) else None


def has_converter(converters: list, name: str) -> bool:
    canon = _canonical(name)
    return any(_name_of(c) == canon for c in converters)


def active_plan_updaters() -> list[type[PlanUpdater]]:
    return list(_ACTIVE_PLAN_UPDATERS)


def active_state_dict_updaters() -> list[type[StateDictUpdater]]:
    return list(_ACTIVE_SD_UPDATERS)


def reset_active_converters() -> None:
    _ACTIVE_PLAN_UPDATERS.clear()
    _ACTIVE_SD_UPDATERS.clear()


class ModelConvertersContainer:
    """Runs the listed converters in order; order matters (e.g. grouped-GEMM before MXFP8)."""

    def __init__(self, converters: list, *, model_spec=None, trainer_config=None):
        _ensure_discovered()
        reset_active_converters()
        self.entries: list[tuple[ConverterSpec | None, Any]] = []
        for entry in converters:
            if hasattr(entry, "build") and not isinstance(entry, (str, ConverterConfig)):
                # a self-contained converter config (e.g. MXFP8Converter.Config)
                self.entries.append((None, entry.build(model_spec=model_spec, trainer_config=trainer_config)))
                continue
            name = _name_of(entry)
            if name is None or name not in _REGISTRY:
                raise KeyError(f"unknown model converter {entry!r}; registered: {sorted(_REGISTRY)}")
            spec = _REGISTRY[name]
            inst = None
            if spec.model_converter is not None:
                inst = spec.model_converter(model_spec, trainer_config)
                if isinstance(entry, ConverterConfig):
                    inst.options = dict(entry.options)
            self.entries.append((spec, inst))

    def convert(self, model: nn.Module) -> None:
        for spec, inst in self.entries:
            if inst is not None:
                inst.convert(model)
            if spec is not None:
                if spec.plan_updater is not None and spec.plan_updater not in _ACTIVE_PLAN_UPDATERS:
                    _ACTIVE_PLAN_UPDATERS.append(spec.plan_updater)
                if spec.state_dict_updater is not None and spec.state_dict_updater not in _ACTIVE_SD_UPDATERS:
                    _ACTIVE_SD_UPDATERS.append(spec.state_dict_updater)

    def post_optimizer_hook(self, model_parts) -> None:
        for _, inst in self.entries:
            if inst is not None and hasattr(inst, "post_optimizer_hook"):
                inst.post_optimizer_hook(model_parts)
