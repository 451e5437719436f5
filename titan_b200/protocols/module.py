"""Module / Config protocol.

Every model building block is described by a dataclass config with a
``build()`` method, so a model can be instantiated on the meta device from a
recipe, mutated by converters, parallelised, and only then materialised
(``to_empty`` + ``init_states``).

Parity: the reference builds all of its models on upstream's
`Module/Module.Config/config.build()/init_states` protocol
(torchtitan_npu/models/deepseek_v32/model.py:37-38,239).
"""

from __future__ import annotations

from dataclasses import dataclass, fields, is_dataclass
from typing import Any, ClassVar

import torch
import torch.nn as nn

__all__ = ["Configurable", "Module", "ModuleDict", "ModuleList", "BaseModelConfig"]


class Configurable:
    """Mixin: a class with a nested ``Config`` dataclass whose ``build()`` constructs it."""

    @dataclass(kw_only=True)
    class Config:
        _owner: ClassVar[type | None] = None

        def build(self, **kwargs):
            owner = type(self)._owner
            if owner is None:
                raise TypeError(f"{type(self).__qualname__} is not bound to a class")
            return owner(self, **kwargs)

        def to_dict(self) -> dict:
            out = {}
            for f in fields(self):
                v = getattr(self, f.name)
                out[f.name] = v.to_dict() if hasattr(v, "to_dict") and is_dataclass(v) else v
            return out

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        cfg = cls.__dict__.get("Config")
        if cfg is not None:
            cfg._owner = cls


class Module(nn.Module, Configurable):
    """`nn.Module` with recursive state initialisation.

    ``init_states`` initialises parameters *and* non-persistent buffers; it is
    called after ``to_empty`` so that a model built on the meta device can be
    materialised shard by shard.
    """

    def init_states(self, *, buffer_device: torch.device | None = None, **kwargs: Any) -> None:
        for child in self.children():
            if isinstance(child, Module):
                child.init_states(buffer_device=buffer_device, **kwargs)
            elif hasattr(child, "reset_parameters"):
                child.reset_parameters()
            else:
                for sub in child.modules():
                    if sub is not child and isinstance(sub, Module):
                        sub.init_states(buffer_device=buffer_device, **kwargs)

    # alias kept for recipes written against the older name
    def init_weights(self, *args, **kwargs) -> None:
        self.init_states(*args, **kwargs)


class ModuleDict(nn.ModuleDict, Module):
    """Dict of blocks keyed by the layer index string, so PP can delete layers without renumbering FQNs."""

    def init_states(self, **kwargs):
        for m in self.values():
            if m is not None and isinstance(m, Module):
                m.init_states(**kwargs)


class ModuleList(nn.ModuleList, Module):
    def init_states(self, **kwargs):
        for m in self:
            if m is not None and isinstance(m, Module):
                m.init_states(**kwargs)


@dataclass(kw_only=True)
class BaseModelConfig(Configurable.Config):
    """Common surface of all model configs."""

    dim: int = 256
    n_layers: int = 2
    vocab_size: int = 2048
    max_seq_len: int = 2048

    def update_from_config(self, *, trainer_config, **kwargs) -> None:
        """Let the model read trainer fields (seq_len, MTP count, converter presence)."""
        self.max_seq_len = max(self.max_seq_len, trainer_config.training.seq_len)

    def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, int]:
        nparams = sum(p.numel() for p in model.parameters())
        return nparams, 6 * nparams
