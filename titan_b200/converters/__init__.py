"""Model converters.  Importing this package imports every converter module so that each
registers itself; RoPE comes first because other converters look up its replaced functions.

Parity: torchtitan_npu/converters/__init__.py:30-48.
"""

import importlib
import pkgutil

_FIRST = ["rope"]


def _discover() -> None:
    names = [m.name for m in pkgutil.iter_modules(__path__) if not m.name.startswith("_")]
    ordered = [n for n in _FIRST if n in names] + [n for n in names if n not in _FIRST]
    for name in ordered:
        importlib.import_module(f"{__name__}.{name}")


_discover()
