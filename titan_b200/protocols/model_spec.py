"""`ModelSpec`: everything the trainer needs to know about one model flavor.

Parity: the reference registers models as
``ModelSpec(name, flavor, model, parallelize_fn, pipelining_fn, build_loss_fn,
post_optimizer_build_fn, state_dict_adapter)``
(torchtitan_npu/models/deepseek_v3/__init__.py:180-192).
"""

from __future__ import annotations

import importlib
from collections.abc import Callable
from dataclasses import dataclass
from typing import Any

__all__ = ["ModelSpec", "get_model_spec", "list_models"]


@dataclass
class ModelSpec:
    name: str
    flavor: str
    model: Any
    """Model config instance (a `BaseModelConfig`); ``model.build()`` constructs the module."""
    parallelize_fn: Callable
    pipelining_fn: Callable | None = None
    build_loss_fn: Callable | None = None
    post_optimizer_build_fn: Callable | None = None
    state_dict_adapter: type | None = None


_SUPPORTED = ["llama3", "qwen3", "deepseek_v3", "deepseek_v32", "deepseek_v4", "vlm"]


def list_models() -> list[str]:
    return list(_SUPPORTED)


def get_model_spec(name: str, flavor: str) -> ModelSpec:
    """Import ``titan_b200.models.<name>`` (or a full path) and ask its ``model_registry``."""
    mod_name = name if "." in name else f"titan_b200.models.{name}"
    mod = importlib.import_module(mod_name)
    if not hasattr(mod, "model_registry"):
        raise AttributeError(f"{mod_name} does not define model_registry(flavor)")
    return mod.model_registry(flavor)
