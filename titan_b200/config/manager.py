"""``--module / --config`` resolution and dotted command-line overrides.

``--module`` names a model package (short name under ``titan_b200.models`` or a
full import path) whose ``config_registry`` module defines recipe functions;
``--config`` names the function.  The function returns a complete
`TrainerConfig`; remaining ``--section.field value`` arguments override single
fields.  Booleans accept ``--section.flag`` / ``--section.no-flag``; list fields
take comma-separated values; hyphens and underscores are interchangeable.

A field whose type is a union of config classes (the data loader: text, chat,
synthetic or multimodal; the chat encoder) is switched with a bare
``section:variant`` token, the variant being the class name in snake case
(``dataloader:chat_data_loader_config``); the section is replaced by that
class's defaults and later ``--section.field`` overrides apply to it, so put
the token before them.

Parity: launch path of the reference (torchtitan_npu/entry.py:31-32,
scripts/run_train.sh:25-39, docs/feature_guides/checkpoint.md:62-73).
"""

from __future__ import annotations

import importlib
import sys
import types
import typing
from dataclasses import fields, is_dataclass
from typing import Any, get_args, get_origin

from titan_b200.config.configs import TrainerConfig

__all__ = ["ConfigManager", "resolve_recipe", "apply_overrides"]


def _import_registry(module: str):
    candidates = []
    if "." in module:
        candidates += [module + ".config_registry", module]
    else:
        candidates += [f"titan_b200.models.{module}.config_registry", f"{module}.config_registry", module]
    last_err: Exception | None = None
    for name in candidates:
        try:
            return importlib.import_module(name)
        except ModuleNotFoundError as e:  # try the next spelling
            # an import error raised *inside* an existing module must surface
            if e.name is not None and not name.startswith(e.name):
                raise
            last_err = e
    raise ModuleNotFoundError(f"cannot resolve --module {module!r}: tried {candidates}") from last_err


def resolve_recipe(module: str, config: str) -> TrainerConfig:
    reg = _import_registry(module)
    if not hasattr(reg, config):
        avail = sorted(n for n, v in vars(reg).items() if callable(v) and not n.startswith("_"))
        raise AttributeError(f"{reg.__name__} has no recipe {config!r}; available: {avail}")
    cfg = getattr(reg, config)()
    if not isinstance(cfg, TrainerConfig):
        raise TypeError(f"recipe {config} returned {type(cfg).__name__}, expected TrainerConfig")
    return cfg


def _strip_optional(tp):
    origin = get_origin(tp)
    if origin is typing.Union or origin is types.UnionType:
        args = [a for a in get_args(tp) if a is not type(None)]
        return args, type(None) in get_args(tp)
    return [tp], False


def _parse_scalar(text: str, tp) -> Any:
    if tp is bool:
        low = text.lower()
        if low in ("1", "true", "yes", "on"):
            return True
        if low in ("0", "false", "no", "off"):
            return False
        raise ValueError(f"not a bool: {text!r}")
    if tp is int:
        return int(text)
    if tp is float:
        return float(text)
    if tp is str or tp is Any:
        return text
    if get_origin(tp) is typing.Literal:
        for choice in get_args(tp):
            if str(choice) == text:
                return choice
        raise ValueError(f"{text!r} not in {get_args(tp)}")
    raise ValueError(f"unsupported scalar type {tp}")


def _parse_value(text: str, tp) -> Any:
    alts, optional = _strip_optional(tp)
    if optional and text.lower() in ("none", "null"):
        return None
    errors = []
    for alt in alts:
        origin = get_origin(alt)
        try:
            if origin in (list, tuple) or alt in (list, tuple):
                inner = get_args(alt)[0] if get_args(alt) else str
                items = [t for t in text.split(",") if t != ""]
                return [_parse_value(t, inner) for t in items]
            if origin is dict or alt is dict:
                import json

                return json.loads(text)
            return _parse_scalar(text, alt)
        except (ValueError, TypeError) as e:
            errors.append(str(e))
    raise ValueError(f"cannot parse {text!r} as {tp}: {errors}")


def _field_types(obj) -> dict[str, Any]:
    hints = typing.get_type_hints(type(obj))
    return {f.name: hints.get(f.name, Any) for f in fields(obj)}


def _lookup(cfg, dotted: str):
    """Return (owner dataclass, field name, field type, negated?) for a dotted key."""
    parts = [p.replace("-", "_") for p in dotted.split(".")]
    obj = cfg
    for p in parts[:-1]:
        if not is_dataclass(obj) or not hasattr(obj, p):
            raise KeyError(f"unknown config section {p!r} in --{dotted}")
        obj = getattr(obj, p)
    leaf = parts[-1]
    types_ = _field_types(obj)
    if leaf in types_:
        return obj, leaf, types_[leaf], False
    if leaf.startswith("no_") and leaf[3:] in types_:
        return obj, leaf[3:], types_[leaf[3:]], True
    raise KeyError(f"unknown config field --{dotted} (section has {sorted(types_)})")


def _snake(name: str) -> str:
    import re

    return re.sub(r"(?<=[a-z0-9])(?=[A-Z])|(?<=[A-Z])(?=[A-Z][a-z])", "_", name).lower()


def _switch_variant(cfg, token: str) -> None:
    """``section[.sub]:variant`` → replace that field with the defaults of the named member of its union type."""
    dotted, _, variant = token.partition(":")
    owner, name, tp, negated = _lookup(cfg, dotted)
    alts, _ = _strip_optional(tp)
    classes = [a for a in alts if isinstance(a, type) and is_dataclass(a)]
    want = variant.replace("-", "_").lower()
    for cls in classes:
        if _snake(cls.__name__) == want or cls.__name__.lower() == want:
            setattr(owner, name, cls())
            return
    raise SystemExit(f"{token!r}: --{dotted} takes one of {[_snake(c.__name__) for c in classes]}")


def apply_overrides(cfg: TrainerConfig, argv: list[str]) -> TrainerConfig:
    """Apply ``--a.b value`` / ``--a.b=value`` / ``--a.flag`` / ``--a.no-flag`` / ``a:variant`` in place."""
    i = 0
    while i < len(argv):
        tok = argv[i]
        if not tok.startswith("--") and ":" in tok:
            _switch_variant(cfg, tok)
            i += 1
            continue
        if not tok.startswith("--"):
            raise SystemExit(f"unexpected argument {tok!r}")
        key, eq, val = tok[2:].partition("=")
        owner, name, tp, negated = _lookup(cfg, key)
        alts, _ = _strip_optional(tp)
        is_bool = alts == [bool]
        if negated:
            if not is_bool:
                raise SystemExit(f"--{key}: 'no-' prefix only applies to boolean fields")
            setattr(owner, name, False)
            i += 1
            continue
        if not eq:
            nxt = argv[i + 1] if i + 1 < len(argv) else None
            if is_bool and (nxt is None or nxt.startswith("--")):
                setattr(owner, name, True)
                i += 1
                continue
            if nxt is None:
                raise SystemExit(f"--{key} needs a value")
            val = nxt
            i += 1
        setattr(owner, name, _parse_value(val, tp))
        i += 1
    return cfg


class ConfigManager:
    """Parses ``--module M --config C [--dotted.overrides ...]`` into a `TrainerConfig`."""

    def parse_args(self, argv: list[str] | None = None) -> TrainerConfig:
        argv = list(sys.argv[1:] if argv is None else argv)
        module = config = None
        rest: list[str] = []
        i = 0
        while i < len(argv):
            tok = argv[i]
            name, eq, val = tok.partition("=")
            if name in ("--module", "--config"):
                if not eq:
                    i += 1
                    val = argv[i]
                if name == "--module":
                    module = val
                else:
                    config = val
            else:
                rest.append(tok)
            i += 1
        if module is None or config is None:
            raise SystemExit("usage: --module <model package> --config <recipe function> [--section.field value ...]")
        cfg = resolve_recipe(module, config)
        return apply_overrides(cfg, rest)
