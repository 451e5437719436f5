"""Supervised fine-tuning loader: chat samples → token sequences with assistant-only labels, packed to ``seq_len``.

Pipeline per raw sample: ``sample_processor`` (or the ``chat_processor`` import path) → messages → validation of the
turn structure (system?, then alternating non-assistant / assistant turns; consecutive user/tool messages count as one
turn, which admits OpenAI-style tool-call transcripts) → chat encoder (tokenizer template + ChatML header scan by
default, or a configured encoder) → ``input = tokens[:-1]``, ``labels = tokens[1:]`` with everything outside the
assistant ranges set to the ignore index.  Samples longer than ``seq_len`` and samples without any supervised token are
dropped.  With ``pack_sequences`` several samples share a row; ``positions`` restart at every sample so that
block-causal / variable-length attention keeps them apart.  A row is padded with EOS inputs and ignored labels.

Rows come from a local JSON / JSON-lines / parquet file (``data_files`` or ``dataset_path`` pointing at a file or
folder) through the `datasets` library, or from any iterable handed to `ChatDataLoader(samples=...)`.

Parity: upstream `ChatDataset` / `ChatDataLoader` with the reference's patches
(torchtitan_npu/patches/torchtitan/chat_dataset.py:24-292: loader-config preparation, multi-turn validation,
encoder routing, assistant-range label masking, MTP sequence extension).
"""

from __future__ import annotations

import os
from collections.abc import Iterable
from typing import Any

import torch

from titan_b200.data.chat_encoders import BaseChatEncoder, ChatMLEncoder, build_chat_encoder
from titan_b200.data.chat_processors import import_chat_processor
from titan_b200.utils.logging import logger

__all__ = ["validate_messages", "labels_for_token_ranges", "ChatDataLoader", "build_chat_dataloader"]

IGNORE_INDEX = -100
_VALID_ROLES = {"assistant", "system", "tool", "user"}


def validate_messages(messages: list[dict[str, Any]]) -> None:
    if len(messages) < 2:
        raise ValueError(f"Expected at least 2 messages, got {len(messages)}")
    for i, m in enumerate(messages):
        if m.get("role") not in _VALID_ROLES:
            raise ValueError(f"Unknown role '{m.get('role')}' at index {i}")
    if len(messages) == 2:
        if messages[0].get("role") != "user":
            raise ValueError(f"First message must be 'user', got '{messages[0].get('role')}'")
        if messages[1].get("role") != "assistant":
            raise ValueError(f"Second message must be 'assistant', got '{messages[1].get('role')}'")
        return
    if messages[0].get("role") not in ("system", "user"):
        raise ValueError(f"First message must be 'user' or 'system', got '{messages[0].get('role')}'")
    start = 1 if messages[0].get("role") == "system" else 0
    rest = messages[start:]
    if len(rest) < 2:
        raise ValueError("Need at least one (non-assistant, assistant) pair after system")
    turns: list[tuple[int, dict]] = []  # runs of non-assistant messages collapse into one turn
    for i, m in enumerate(rest):
        if m.get("role") != "assistant" and turns and turns[-1][1].get("role") != "assistant":
            turns[-1] = (start + i, m)
        else:
            turns.append((start + i, m))
    for j in range(0, len(turns), 2):
        idx, m = turns[j]
        if m.get("role") == "assistant":
            raise ValueError(f"Expected non-assistant at position {idx}, got 'assistant'")
        if j + 1 < len(turns) and turns[j + 1][1].get("role") != "assistant":
            raise ValueError(f"Expected 'assistant' at position {turns[j + 1][0]}, got "
                             f"'{turns[j + 1][1].get('role')}'")


def labels_for_token_ranges(label_ids: list[int], token_ranges) -> list[int]:
    """``label_ids[i]`` is ``tokens[i + 1]``: a token range ``[s, e)`` supervises labels ``[s - 1, e - 1)``."""
    out = [IGNORE_INDEX] * len(label_ids)
    for s, e in token_ranges:
        for i in range(max(s - 1, 0), min(e - 1, len(label_ids))):
            out[i] = label_ids[i]
    return out


def _load_rows(cfg) -> Iterable:
    kwargs = dict(cfg.load_dataset_kwargs or {})
    if cfg.dataset_split:
        kwargs["split"] = cfg.dataset_split
    if cfg.data_files:
        kwargs["data_files"] = cfg.data_files
    if cfg.dataset_config_name:
        kwargs["name"] = cfg.dataset_config_name
    kwargs = {k: v for k, v in kwargs.items() if v not in (None, "")}
    from datasets import load_dataset

    path = cfg.dataset_path
    files = kwargs.get("data_files") or (path if path and os.path.isfile(path) else None)
    if files:
        ext = str(files).rsplit(".", 1)[-1].lower()
        builder = {"jsonl": "json", "json": "json", "parquet": "parquet", "csv": "csv"}.get(ext, "json")
        kwargs.pop("name", None)
        return load_dataset(builder, data_files=files, split=kwargs.get("split", "train"))
    if path and os.path.isdir(path):
        return load_dataset(path, **kwargs)
    raise FileNotFoundError(f"chat dataset {path!r}: pass a local file or folder (dataset_path / data_files); hub "
                            "names cannot be fetched without network access")


class ChatDataLoader:
    def __init__(self, cfg=None, *, tokenizer, seq_len: int, batch_size: int, dp_rank: int = 0,
                 dp_world_size: int = 1, samples: Iterable | None = None, sample_processor=None,
                 chat_encoder: BaseChatEncoder | None = None, extra_tokens: int = 0, pack_sequences: bool = True,
                 infinite: bool = True, pin_memory: bool = True):
        if tokenizer is None or tokenizer.eos_id is None:
            raise ValueError("a chat dataloader needs a tokenizer with an EOS id")
        self.tok, self.eos_id = tokenizer, tokenizer.eos_id
        self.seq_len, self.batch_size, self.extra = seq_len + extra_tokens, batch_size, extra_tokens
        self.dp_rank, self.dp_world_size = dp_rank, dp_world_size
        self.pack, self.infinite = pack_sequences, infinite
        self.pin = pin_memory and torch.cuda.is_available()
        if cfg is not None:
            sample_processor = sample_processor or cfg.sample_processor
            if cfg.chat_processor:
                sample_processor = import_chat_processor(cfg.chat_processor)
            chat_encoder = chat_encoder or build_chat_encoder(cfg.chat_encoder)
            self.pack, self.infinite = cfg.pack_sequences, cfg.infinite
        if sample_processor is None:
            raise ValueError("ChatDataLoaderConfig requires either sample_processor or chat_processor import path.")
        self._process = sample_processor
        self._encoder = chat_encoder or ChatMLEncoder()
        self._rows = samples if samples is not None else _load_rows(cfg)
        self._sample_idx = 0
        self._logged = False
        self.dropped_long = self.dropped_unsupervised = 0

    # ---- one sample -------------------------------------------------------------------------------------------
    def tokenize_sample(self, sample):
        messages = self._process(sample)
        validate_messages(messages)
        text, tokens, ranges = self._encoder.encode_messages_with_assistant_ranges(messages, self.tok, self.eos_id)
        if not self._logged:
            logger.info("first chat sample (%d chars, %d tokens):\n--- HEAD ---\n%s\n--- TAIL ---\n%s", len(text),
                        len(tokens), text[:500], text[-500:])
            self._logged = True
        if len(tokens) - 1 > self.seq_len:
            self.dropped_long += 1
            return None
        inputs, labels = tokens[:-1], labels_for_token_ranges(tokens[1:], ranges)
        if all(v == IGNORE_INDEX for v in labels):
            self.dropped_unsupervised += 1
            logger.warning("dropping sample %d: all labels are masked; check assistant spans and chat template",
                           self._sample_idx)
            return None
        return inputs, labels

    def _stream(self):
        while True:
            seen = 0
            for i, row in enumerate(self._rows):
                if i % self.dp_world_size != self.dp_rank:
                    continue
                seen += 1
                if seen <= self._sample_idx:
                    continue
                self._sample_idx = seen
                out = self.tokenize_sample(row)
                if out is not None:
                    yield out
            if not self.infinite:
                return
            if seen == 0:
                raise RuntimeError("the chat dataset has no rows for this data-parallel rank")
            self._sample_idx = 0

    def _rows_packed(self):
        inp: list[int] = []
        lab: list[int] = []
        pos: list[int] = []
        for a, b in self._stream():
            if inp and (not self.pack or len(inp) + len(a) > self.seq_len):
                yield self._pad(inp, lab, pos)
                inp, lab, pos = [], [], []
            inp += a
            lab += b
            pos += list(range(len(a)))
        if inp:
            yield self._pad(inp, lab, pos)

    def _pad(self, inp, lab, pos):
        n = self.seq_len - len(inp)
        return (torch.tensor(inp + [self.eos_id] * n), torch.tensor(lab + [IGNORE_INDEX] * n),
                torch.tensor(pos + list(range(n))))

    def __iter__(self):
        rows = []
        for r in self._rows_packed():
            rows.append(r)
            if len(rows) == self.batch_size:
                inputs, labels, positions = (torch.stack(x) for x in zip(*rows))
                rows = []
                # rows are seq_len + extra long: MTP depth k reads inputs[:, k : k + seq_len] and labels[:, k : ...];
                # positions describe the seq_len main tokens
                batch = {"input": inputs, "positions": positions[:, : self.seq_len - self.extra]}
                if self.pin:
                    batch = {k: v.pin_memory() for k, v in batch.items()}
                    labels = labels.pin_memory()
                yield batch, labels

    def state_dict(self) -> dict[str, Any]:
        return {"sample_idx": self._sample_idx, "dp_world_size": self.dp_world_size}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        if sd:
            self._sample_idx = int(sd["sample_idx"])


def build_chat_dataloader(cfg, *, tokenizer, training, dp_rank: int, dp_world_size: int) -> ChatDataLoader:
    return ChatDataLoader(cfg, tokenizer=tokenizer, seq_len=training.seq_len, batch_size=training.local_batch_size,
                          dp_rank=dp_rank, dp_world_size=dp_world_size, extra_tokens=training.num_mtp_modules,
                          pin_memory=cfg.pin_memory)
