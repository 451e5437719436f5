"""Tokenizers.

* `HFTokenizer` – reads a Hugging Face asset folder (``tokenizer.json``, or ``vocab.json`` + ``merges.txt``;
  ``tokenizer_config.json`` for BOS/EOS and the chat template) through the `tokenizers` library; chat templates
  are rendered with jinja2.
* `ByteTokenizer` – 256 byte ids + a few specials, no files: for tests and dry runs.

Both expose ``encode(text, add_bos, add_eos)``, ``decode(ids)``, ``bos_id``, ``eos_id``, ``vocab_size`` and
``apply_chat_template(messages, tokenize=False)`` (ChatML when the assets carry no template).

Parity: the upstream `HuggingFaceTokenizer` the reference builds from ``hf_assets_path`` (recipes in
torchtitan_npu/models/*/config_registry.py set it; tests/assets/tokenizer/* are such folders).
"""

from __future__ import annotations

import json
import os
from typing import Any

__all__ = ["BaseTokenizer", "HFTokenizer", "ByteTokenizer", "build_tokenizer", "render_chatml"]


def render_chatml(messages: list[dict[str, Any]], add_generation_prompt: bool = False) -> str:
    """``<|im_start|>role\\ncontent<|im_end|>\\n`` per message; assistant reasoning goes into a ``<think>`` block."""
    out = []
    for m in messages:
        content = m.get("content") or ""
        if m.get("role") == "assistant" and m.get("reasoning_content"):
            content = f"<think>\n{m['reasoning_content']}\n</think>\n\n{content}"
        out.append(f"<|im_start|>{m['role']}\n{content}<|im_end|>\n")
    if add_generation_prompt:
        out.append("<|im_start|>assistant\n")
    return "".join(out)


class BaseTokenizer:
    bos_id: int | None = None
    eos_id: int | None = None
    pad_id: int | None = None
    chat_template: str | None = None

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False) -> list[int]:
        raise NotImplementedError

    def decode(self, ids) -> str:
        raise NotImplementedError

    @property
    def vocab_size(self) -> int:
        raise NotImplementedError

    def _wrap(self, ids: list[int], add_bos: bool, add_eos: bool) -> list[int]:
        if add_bos and self.bos_id is not None and (not ids or ids[0] != self.bos_id):
            ids = [self.bos_id] + ids
        if add_eos and self.eos_id is not None and (not ids or ids[-1] != self.eos_id):
            ids = ids + [self.eos_id]
        return ids

    def apply_chat_template(self, messages, tokenize: bool = False, add_generation_prompt: bool = False, **kw):
        if self.chat_template:
            import jinja2

            env = jinja2.Environment(loader=jinja2.BaseLoader(), trim_blocks=True, lstrip_blocks=True)
            env.globals["raise_exception"] = lambda msg: (_ for _ in ()).throw(ValueError(msg))
            text = env.from_string(self.chat_template).render(
                messages=messages, add_generation_prompt=add_generation_prompt,
                bos_token=getattr(self, "bos_token", "") or "", eos_token=getattr(self, "eos_token", "") or "", **kw)
        else:
            text = render_chatml(messages, add_generation_prompt)
        return self.encode(text, add_bos=False, add_eos=False) if tokenize else text


class HFTokenizer(BaseTokenizer):
    def __init__(self, path: str):
        from tokenizers import Tokenizer

        self.path = path
        tj = os.path.join(path, "tokenizer.json")
        if os.path.exists(tj):
            self.tok = Tokenizer.from_file(tj)
        elif os.path.exists(os.path.join(path, "vocab.json")) and os.path.exists(os.path.join(path, "merges.txt")):
            from tokenizers import decoders, models, pre_tokenizers

            self.tok = Tokenizer(models.BPE.from_file(os.path.join(path, "vocab.json"),
                                                      os.path.join(path, "merges.txt")))
            self.tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
            self.tok.decoder = decoders.ByteLevel()
        else:
            raise FileNotFoundError(f"no tokenizer.json or vocab.json + merges.txt under {path!r}")
        cfg = {}
        cj = os.path.join(path, "tokenizer_config.json")
        if os.path.exists(cj):
            with open(cj) as f:
                cfg = json.load(f)
        added = cfg.get("added_tokens_decoder") or {}
        if added and not os.path.exists(tj):
            from tokenizers import AddedToken

            self.tok.add_special_tokens([AddedToken(v["content"], special=True) for _, v in
                                         sorted(added.items(), key=lambda kv: int(kv[0]))])
        self.bos_token = self._tok_str(cfg.get("bos_token"))
        self.eos_token = self._tok_str(cfg.get("eos_token"))
        self.pad_token = self._tok_str(cfg.get("pad_token"))
        self.bos_id = self.tok.token_to_id(self.bos_token) if self.bos_token else None
        self.eos_id = self.tok.token_to_id(self.eos_token) if self.eos_token else None
        self.pad_id = self.tok.token_to_id(self.pad_token) if self.pad_token else None
        self.chat_template = cfg.get("chat_template")
        self.add_bos_default = bool(cfg.get("add_bos_token", False))

    @staticmethod
    def _tok_str(v):
        return v.get("content") if isinstance(v, dict) else v

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False) -> list[int]:
        ids = self.tok.encode(text, add_special_tokens=False).ids
        return self._wrap(ids, add_bos, add_eos)

    def decode(self, ids) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=False)

    @property
    def vocab_size(self) -> int:
        return self.tok.get_vocab_size(with_added_tokens=True)


class ByteTokenizer(BaseTokenizer):
    """ids 0..255 = bytes; 256 = BOS, 257 = EOS, 258 = PAD, then the ChatML markers as single tokens."""

    SPECIALS = ("<|bos|>", "<|eos|>", "<|pad|>", "<|im_start|>", "<|im_end|>")

    def __init__(self):
        self.bos_id, self.eos_id, self.pad_id = 256, 257, 258
        self.bos_token, self.eos_token = self.SPECIALS[0], self.SPECIALS[1]
        self._sp = {s: 256 + i for i, s in enumerate(self.SPECIALS)}

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False) -> list[int]:
        ids: list[int] = []
        i = 0
        while i < len(text):
            for s, tid in self._sp.items():
                if text.startswith(s, i):
                    ids.append(tid)
                    i += len(s)
                    break
            else:
                j = i + 1
                while j < len(text) and not any(text.startswith(s, j) for s in self._sp):
                    j += 1
                ids.extend(text[i:j].encode("utf-8"))
                i = j
        return self._wrap(ids, add_bos, add_eos)

    def decode(self, ids) -> str:
        inv = {v: k for k, v in self._sp.items()}
        out, buf = [], bytearray()
        for t in ids:
            if t < 256:
                buf.append(t)
            else:
                out.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
                out.append(inv.get(int(t), ""))
        out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)

    @property
    def vocab_size(self) -> int:
        return 256 + len(self.SPECIALS)


def build_tokenizer(path: str | None) -> BaseTokenizer:
    """A folder with tokenizer files → `HFTokenizer`; ``"byte"`` → `ByteTokenizer`."""
    if path in ("byte", "bytes"):
        return ByteTokenizer()
    if path and os.path.isdir(path):
        return HFTokenizer(path)
    raise FileNotFoundError(f"tokenizer assets not found at {path!r} (pass a Hugging Face asset folder, or 'byte' for "
                            "the file-less byte tokenizer)")
