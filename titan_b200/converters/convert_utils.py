"""Helpers converters use to rewrite a model in place.

* `find_modules / replace_modules` – match on the class name (regex) and swap instances, keeping
  parameters and attributes (the new instance shares ``__dict__`` where asked to).
* `find_functions / replace_functions` – rebind a free function everywhere it was imported: a
  ``from pkg import f`` creates a second binding in the importing module, so patching ``pkg.f``
  alone misses it; every loaded module of this package is scanned for the old object.
* `replace_methods` – set a method on every matching class.
* `replace_module_with_name` – swap one submodule by its dotted path.

Parity: torchtitan_npu/converters/convert_utils.py:18-180.
"""

from __future__ import annotations

import re
import sys
from collections.abc import Callable

import torch.nn as nn

__all__ = [
    "find_modules",
    "replace_modules",
    "find_functions",
    "replace_functions",
    "find_methods",
    "replace_methods",
    "replace_module_with_name",
]


def find_modules(model: nn.Module, class_pattern: str) -> list[tuple[str, nn.Module]]:
    rx = re.compile(class_pattern)
    return [(n, m) for n, m in model.named_modules() if rx.fullmatch(type(m).__name__)]


def replace_module_with_name(model: nn.Module, name: str, new: nn.Module) -> None:
    parent_name, _, leaf = name.rpartition(".")
    parent = model.get_submodule(parent_name) if parent_name else model
    parent.register_module(leaf, new)


def replace_modules(model: nn.Module, class_pattern: str, factory: Callable[[nn.Module], nn.Module]) -> int:
    """Replace every module whose class name matches; `factory(old) -> new`.  Returns the count."""
    hits = [(n, m) for n, m in find_modules(model, class_pattern) if n != ""]
    for name, mod in hits:
        replace_module_with_name(model, name, factory(mod))
    return len(hits)


def _package_modules(prefixes: tuple[str, ...]):
    for name, mod in list(sys.modules.items()):
        if mod is not None and name.startswith(prefixes):
            yield name, mod


def find_functions(func: Callable, prefixes: tuple[str, ...] = ("titan_b200",)) -> list[tuple[str, str]]:
    """All (module name, attribute name) bindings of `func` in loaded modules of the package."""
    out = []
    for name, mod in _package_modules(prefixes):
        for attr, val in list(vars(mod).items()):
            if val is func:
                out.append((name, attr))
    return out


def replace_functions(old: Callable, new: Callable, prefixes: tuple[str, ...] = ("titan_b200",),
                      skip_modules: tuple[str, ...] = ()) -> int:
    n = 0
    for mod_name, attr in find_functions(old, prefixes):
        if mod_name.startswith(skip_modules) if skip_modules else False:
            continue
        setattr(sys.modules[mod_name], attr, new)
        n += 1
    return n


def find_methods(model: nn.Module, class_pattern: str, method: str) -> list[type]:
    rx = re.compile(class_pattern)
    seen: list[type] = []
    for m in model.modules():
        cls = type(m)
        if rx.fullmatch(cls.__name__) and hasattr(cls, method) and cls not in seen:
            seen.append(cls)
    return seen


def replace_methods(model: nn.Module, class_pattern: str, method: str, new: Callable) -> int:
    classes = find_methods(model, class_pattern, method)
    for cls in classes:
        setattr(cls, method, new)
    return len(classes)
