"""The documentation names real things: every ``--section.field`` flag, every ``section:variant`` token, every recipe
and every repository path mentioned in `docs/`, `README.md` and `examples/` must exist."""

import glob
import os
import re

import pytest

from titan_b200.config.configs import TrainerConfig
from titan_b200.config.manager import _lookup, _switch_variant

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FILES = sorted(glob.glob(os.path.join(ROOT, "docs", "**", "*.md"), recursive=True)
               + glob.glob(os.path.join(ROOT, "examples", "*", "*"))
               + [os.path.join(ROOT, "README.md")])
FLAG = re.compile(r"--([a-z_]+(?:\.[a-z_0-9-]+)+)")
VARIANT = re.compile(r"(?<![\w/.-])((?:dataloader|dataloader\.chat_encoder):[a-z_0-9]+)")
PATH = re.compile(r"`((?:titan_b200|scripts|tests|benchmarks|examples|profiles|docs)/[\w./*{},-]+)`")


def _fresh():
    """One configuration per data-loader kind (flags of a kind only exist once the section is switched to it); the chat
    one comes second."""
    from titan_b200.config import configs as C

    out = []
    for kind in (C.SyntheticDataLoaderConfig, C.ChatDataLoaderConfig, C.TextDataLoaderConfig, C.MultiModalDataLoaderConfig):
        cfg = TrainerConfig()
        cfg.dataloader = kind()
        out.append(cfg)
    return out


@pytest.mark.parametrize("path", FILES, ids=[os.path.relpath(f, ROOT) for f in FILES])
def test_flags_variants_and_paths_exist(path):
    text = open(path, errors="replace").read()
    candidates = _fresh()
    chat = candidates[1]
    for flag in sorted(set(FLAG.findall(text))):
        if flag.split(".")[0] in ("nproc", "master", "local", "nnodes", "node", "section", "a"):  # torchrun / placeholders
            continue
        for candidate in candidates:
            try:
                _lookup(candidate, flag)
                break
            except KeyError:
                continue
        else:
            if flag.startswith("dataloader.chat_encoder."):  # fields of the DSV4 encoder variant
                _switch_variant(chat, "dataloader.chat_encoder:dsv4_encoder_config")
                _lookup(chat, flag)
                continue
            raise AssertionError(f"{os.path.relpath(path, ROOT)} names --{flag}, which is not a config field")
    for token in sorted(set(VARIANT.findall(text))):
        _switch_variant(_fresh()[1], token)
    for ref in sorted(set(PATH.findall(text))):
        if any(ch in ref for ch in "*{"):
            continue
        target = os.path.join(ROOT, ref.rstrip(".,"))
        assert os.path.exists(target), f"{os.path.relpath(path, ROOT)} names `{ref}`, which does not exist"


def test_recipes_named_in_docs_resolve():
    from titan_b200.config.manager import resolve_recipe

    named = set()
    for path in FILES:
        named.update(re.findall(r"MODULE=(\w+) CONFIG=(?:\$\{CONFIG:-)?(\w+)", open(path, errors="replace").read()))
    assert len(named) >= 8
    for module, recipe in sorted(named):
        resolve_recipe(module, recipe)
