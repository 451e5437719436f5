"""Sample → chat-messages processors for SFT datasets, and the import helper that resolves a processor path.

A processor maps one raw dataset row to ``[{"role": ..., "content": ...}, ...]`` (assistant turns may carry
``reasoning_content``; a leading system message may carry ``tools``).

Parity: torchtitan_npu/hf_datasets/chat_processors.py:7-84.
"""

from __future__ import annotations

import json
from collections.abc import Callable
from importlib import import_module

__all__ = ["process_tau_sample", "process_gsm8k_sample", "process_wordle_sample", "process_yelp_sample",
           "import_chat_processor"]

_YELP_STAR_NAMES = ("1 star", "2 stars", "3 stars", "4 stars", "5 stars")


def process_tau_sample(sample):
    """Tool-use transcripts: ``messages`` (JSON string or list) + optional ``tools`` attached to the system turn."""
    raw = sample["messages"]
    messages = [dict(m) for m in (json.loads(raw) if isinstance(raw, str) else raw)]
    raw_tools = sample.get("tools", [])
    tools = json.loads(raw_tools) if isinstance(raw_tools, str) else raw_tools
    if tools:
        if messages and messages[0].get("role") == "system":
            messages[0] = {**messages[0], "tools": tools}
        else:
            messages.insert(0, {"role": "system", "content": "", "tools": tools})
    return messages


def process_gsm8k_sample(sample):
    """``answer`` = worked solution + ``#### final``: the solution becomes the reasoning, the final number the reply."""
    reasoning, final = sample["answer"].rsplit("####", 1)
    return [{"role": "user", "content": sample["question"]},
            {"role": "assistant", "reasoning_content": reasoning.strip(), "content": final.strip()}]


def process_wordle_sample(sample: dict) -> list[dict]:
    if "messages" in sample:
        messages = list(sample["messages"])
    elif "prompt" in sample and "completion" in sample:
        messages = list(sample["prompt"]) + list(sample["completion"])
    else:
        raise KeyError(f"Wordle sample must have 'messages' or 'prompt'+'completion'. Got keys: {list(sample.keys())}")
    out = []
    for m in messages:
        m = dict(m)
        if isinstance(m.get("content"), list):
            m["content"] = "\n".join(str(x) for x in m["content"])
        out.append(m)
    return out


def process_yelp_sample(sample):
    text = str(sample.get("text", "")).strip()
    return [{"role": "user", "content": "Classify the sentiment of the following review by its star rating from 1 to 5 "
                                        f"stars.\n\nReview: {text}"},
            {"role": "assistant", "content": _YELP_STAR_NAMES[int(sample["label"])]}]


def import_chat_processor(path: str) -> Callable:
    """``pkg.module:function`` or ``pkg.module.function`` → the callable."""
    module_name, sep, attr = path.partition(":")
    if not sep:
        module_name, _, attr = path.rpartition(".")
    if not module_name or not attr:
        raise ValueError("chat_processor must be an import path like "
                         f"'titan_b200.data.chat_processors:process_gsm8k_sample', got {path!r}")
    module = import_module(module_name)
    try:
        fn = getattr(module, attr)
    except AttributeError as exc:
        raise ValueError(f"Unknown chat_processor import path {path!r}") from exc
    if not callable(fn):
        raise TypeError(f"chat_processor import path {path!r} resolved to non-callable {fn!r}")
    return fn
