"""Row → chat-messages processors for SFT datasets.

A processor turns one raw dataset row into ``[{"role": ..., "content": ...}, ...]`` (assistant turns may carry
``reasoning_content``; a leading system message may carry ``tools``).  The built-in ones live in a small registry
(`PROCESSORS`: short name → function); a recipe names a processor either by that short name or by an import path
(``pkg.module:function`` / ``pkg.module.function``), resolved by `import_chat_processor`.

Parity: torchtitan_npu/hf_datasets/chat_processors.py:7-84 (same row formats and output schema).
"""

from __future__ import annotations

import json
from collections.abc import Callable
from importlib import import_module

__all__ = ["PROCESSORS", "register_processor", "process_tau_sample", "process_gsm8k_sample",
           "process_wordle_sample", "process_yelp_sample", "import_chat_processor"]

PROCESSORS: dict[str, Callable] = {}
_STARS = tuple(f"{n} star{'s' if n > 1 else ''}" for n in range(1, 6))
_YELP_PROMPT = "Classify the sentiment of the following review by its star rating from 1 to 5 stars.\n\nReview: {}"


def register_processor(name: str):
    def deco(fn):
        PROCESSORS[name] = fn
        return fn

    return deco


def _maybe_json(value):
    return json.loads(value) if isinstance(value, str) else value


@register_processor("tau")
def process_tau_sample(sample):
    """Tool-use transcripts: ``messages`` (JSON string or list); ``tools``, when present, ride on the system turn (one
    is created in front when the transcript has none)."""
    messages = [dict(m) for m in _maybe_json(sample["messages"])]
    tools = _maybe_json(sample.get("tools", []))
    if not tools:
        return messages
    has_system = bool(messages) and messages[0].get("role") == "system"
    head = dict(messages[0]) if has_system else {"role": "system", "content": ""}
    head["tools"] = tools
    return [head, *messages[1 if has_system else 0:]]


@register_processor("gsm8k")
def process_gsm8k_sample(sample):
    """``answer`` = worked solution + ``#### final``: the solution becomes the reasoning, the final number the reply."""
    reasoning, _, final = sample["answer"].rpartition("####")
    return [{"role": "user", "content": sample["question"]},
            {"role": "assistant", "reasoning_content": reasoning.strip(), "content": final.strip()}]


def _flat_content(message) -> dict:
    m = dict(message)
    if isinstance(m.get("content"), list):   # multi-part content → one text block
        m["content"] = "\n".join(map(str, m["content"]))
    return m


@register_processor("wordle")
def process_wordle_sample(sample: dict) -> list[dict]:
    """Either a ready ``messages`` list or a ``prompt`` + ``completion`` pair of message lists."""
    if "messages" in sample:
        turns = sample["messages"]
    elif {"prompt", "completion"} <= sample.keys():
        turns = [*sample["prompt"], *sample["completion"]]
    else:
        raise KeyError(f"a wordle row needs `messages`, or `prompt` and `completion`; this one has {sorted(sample)}")
    return [_flat_content(m) for m in turns]


@register_processor("yelp")
def process_yelp_sample(sample):
    review = str(sample.get("text", "")).strip()
    return [{"role": "user", "content": _YELP_PROMPT.format(review)},
            {"role": "assistant", "content": _STARS[int(sample["label"])]}]


def import_chat_processor(path: str) -> Callable:
    """A registered short name, ``pkg.module:function`` or ``pkg.module.function`` → the callable."""
    if path in PROCESSORS:
        return PROCESSORS[path]
    module_name, attr = path.split(":", 1) if ":" in path else (path.rpartition(".")[0], path.rpartition(".")[2])
    if not module_name or not attr:
        raise ValueError(f"{path!r} names no chat processor: use one of {sorted(PROCESSORS)} or an import path such as "
                         "'titan_b200.data.chat_processors:process_gsm8k_sample'")
    fn = getattr(import_module(module_name), attr, None)
    if fn is None:
        raise ValueError(f"module {module_name!r} has no attribute {attr!r} (chat processor {path!r})")
    if not callable(fn):
        raise TypeError(f"chat processor {path!r} is a {type(fn).__name__}, not a function")
    return fn
