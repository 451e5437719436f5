"""Parameter filters for the parameter-level quantisation: small predicates ``(fqn, parameter, module) -> bool`` and
combinators to build the selection a recipe wants ("every expert matrix and every attention projection, but not the
router").  `quantize_params` accepts either such a three-argument filter or a plain ``(fqn, parameter)`` callable.

Parity: experiments/ao_npu/torchao_npu/quantization/filters.py:13-136.
"""

from __future__ import annotations

import inspect
import re
from collections.abc import Callable, Iterable

import torch.nn as nn

__all__ = ["ParamFilter", "match_module_type", "match_fqn_suffix", "match_fqn_exact", "match_fqn_regex", "is_expert",
           "min_dims", "all_filters", "any_filter", "not_filter", "call_filter"]

ParamFilter = Callable[[str, nn.Parameter, nn.Module], bool]


def match_module_type(*types: type) -> ParamFilter:
    """Parameters owned DIRECTLY by a module of one of ``types``."""
    return lambda fqn, p, mod: isinstance(mod, types)


def match_fqn_suffix(suffixes: str | Iterable[str]) -> ParamFilter:
    sfx = (suffixes,) if isinstance(suffixes, str) else tuple(suffixes)
    return lambda fqn, p, mod: fqn.endswith(sfx)


def match_fqn_exact(names: str | Iterable[str]) -> ParamFilter:
    want = {names} if isinstance(names, str) else set(names)
    return lambda fqn, p, mod: fqn in want


def match_fqn_regex(pattern: str) -> ParamFilter:
    rx = re.compile(pattern)
    return lambda fqn, p, mod: rx.search(fqn) is not None


def is_expert() -> ParamFilter:
    """Stacked expert matrices: 3-D ``w1 / w2 / w3 / w13`` of a grouped-experts module."""
    return lambda fqn, p, mod: p.dim() == 3 and fqn.rsplit(".", 1)[-1] in ("w1", "w2", "w3", "w13")


def min_dims(n: int) -> ParamFilter:
    return lambda fqn, p, mod: p.dim() >= n


def all_filters(*filters: ParamFilter) -> ParamFilter:
    return lambda fqn, p, mod: all(call_filter(f, fqn, p, mod) for f in filters)


def any_filter(*filters: ParamFilter) -> ParamFilter:
    return lambda fqn, p, mod: any(call_filter(f, fqn, p, mod) for f in filters)


def not_filter(f: ParamFilter) -> ParamFilter:
    return lambda fqn, p, mod: not call_filter(f, fqn, p, mod)


def call_filter(f: Callable, fqn: str, p: nn.Parameter, mod: nn.Module) -> bool:
    """Call a two- or three-argument filter."""
    try:
        n = len(inspect.signature(f).parameters)
    except (TypeError, ValueError):
        n = 3
    return bool(f(fqn, p, mod) if n >= 3 else f(fqn, p))
