"""Pre-training text loader: documents → tokens → fixed-length packed samples.

A dataset is a registry entry ``name → (loader(path) → iterable of samples, text_of(sample) → str)``.  Built in:
``c4`` / ``c4_test`` / ``c4_validation`` read JSON-lines (``{"text": ...}``) or a `datasets` folder from
``dataset_path``; ``text`` reads plain ``.txt`` files (one document per file or per blank-line block);
``enwiki-eod`` (encyclopedia articles, one per sample, each closed by the end-of-document token) and ``alpaca``
(instruction / input / output records rendered with the Alpaca prompt, or their ready-made ``text`` column) read the
same file formats and default to ``tests/assets/enwiki`` / ``tests/assets/alpaca`` when no path is given.  Documents are
sharded round-robin over data-parallel ranks, tokenised with BOS/EOS, concatenated into a token buffer and cut into
``seq_len + 1 + extra`` windows (``extra`` = MTP look-ahead tokens); the position inside the stream (sample index and
leftover token buffer) is checkpointed, so a resumed run sees the continuation of the same stream.

Parity: the upstream `HuggingFaceTextDataLoader` with the reference's extra datasets and MTP sequence-length
extension (torchtitan_npu/patches/torchtitan/hf_datasets.py:35-121).
"""

from __future__ import annotations

import glob
import json
import os
from collections.abc import Callable, Iterable
from typing import Any

import torch

__all__ = ["register_text_dataset", "TextDataLoader", "build_text_dataloader"]

_REGISTRY: dict[str, tuple[Callable[[str | None], Iterable], Callable[[Any], str]]] = {}


def register_text_dataset(name: str, loader: Callable[[str | None], Iterable], text_of: Callable[[Any], str]):
    _REGISTRY[name] = (loader, text_of)


def _jsonl_or_hf(split: str, default_path: str | None = None):
    def load(path: str | None):
        path = path or default_path
        if not path:
            raise FileNotFoundError("dataloader.dataset_path is required (there is no network access to a hub)")
        files = sorted(glob.glob(os.path.join(path, "**", "*.jsonl"), recursive=True) +
                       glob.glob(os.path.join(path, "**", "*.json"), recursive=True)) if os.path.isdir(path) else [path]
        if files and all(f.endswith((".jsonl", ".json")) for f in files):
            def gen():
                for f in files:
                    with open(f) as fh:
                        for line in fh:
                            line = line.strip()
                            if line:
                                yield json.loads(line)
            return gen()
        from datasets import load_dataset  # a saved `datasets` folder (arrow / parquet)

        return load_dataset(path, split=split, streaming=True)
    return load


def _txt(path: str | None):
    if not path:
        raise FileNotFoundError("dataloader.dataset_path is required")
    files = sorted(glob.glob(os.path.join(path, "**", "*.txt"), recursive=True)) if os.path.isdir(path) else [path]

    def gen():
        for f in files:
            with open(f) as fh:
                for block in fh.read().split("\n\n"):
                    if block.strip():
                        yield {"text": block}
    return gen()


for _name, _split in (("c4", "train"), ("c4_test", "train"), ("c4_validation", "validation")):
    register_text_dataset(_name, _jsonl_or_hf(_split), lambda s: s["text"])
register_text_dataset("text", _txt, lambda s: s["text"])

_ALPACA_WITH_INPUT = ("Below is an instruction that describes a task, paired with an input that provides further "
                      "context. Write a response that appropriately completes the request.\n\n"
                      "### Instruction:\n{instruction}\n\n### Input:\n{input}\n\n### Response:\n{output}")
_ALPACA_NO_INPUT = ("Below is an instruction that describes a task. Write a response that appropriately completes "
                    "the request.\n\n### Instruction:\n{instruction}\n\n### Response:\n{output}")


def _alpaca_text(sample) -> str:
    if sample.get("text"):
        return sample["text"]
    template = _ALPACA_WITH_INPUT if sample.get("input") else _ALPACA_NO_INPUT
    return template.format(instruction=sample.get("instruction", ""), input=sample.get("input", ""),
                           output=sample.get("output", ""))


register_text_dataset("enwiki-eod", _jsonl_or_hf("train", os.path.join("tests", "assets", "enwiki")),
                      lambda s: s["text"])
register_text_dataset("alpaca", _jsonl_or_hf("train", os.path.join("tests", "assets", "alpaca")), _alpaca_text)


class TextDataLoader:
    def __init__(self, *, dataset: str, dataset_path: str | None, tokenizer, seq_len: int, batch_size: int,
                 dp_rank: int, dp_world_size: int, extra_tokens: int = 0, infinite: bool = True,
                 pin_memory: bool = True):
        if dataset not in _REGISTRY:
            raise KeyError(f"unknown text dataset {dataset!r}; registered: {sorted(_REGISTRY)}")
        if tokenizer is None:
            raise ValueError("a text dataloader needs a tokenizer (model.hf_assets_path / model.tokenizer_path)")
        self.dataset, self.path, self.tok = dataset, dataset_path, tokenizer
        self.seq_len, self.batch_size, self.extra = seq_len, batch_size, extra_tokens
        self.dp_rank, self.dp_world_size, self.infinite = dp_rank, dp_world_size, infinite
        self.pin = pin_memory and torch.cuda.is_available()
        self._sample_idx = 0          # documents consumed from the (rank-sharded) stream
        self._epoch = 0
        self._buffer: list[int] = []  # tokens not yet emitted

    def _documents(self):
        loader, text_of = _REGISTRY[self.dataset]
        while True:
            seen = 0
            for i, sample in enumerate(loader(self.path)):
                if i % self.dp_world_size != self.dp_rank:
                    continue
                seen += 1
                if seen <= self._sample_idx:
                    continue  # fast-forward after a resume
                self._sample_idx = seen
                yield text_of(sample)
            if not self.infinite:
                return
            if seen == 0:
                raise RuntimeError(f"dataset {self.dataset!r} at {self.path!r} has no documents for rank {self.dp_rank}")
            self._epoch += 1
            self._sample_idx = 0

    def _samples(self):
        need = self.seq_len + 1 + self.extra
        for text in self._documents():
            self._buffer.extend(self.tok.encode(text, add_bos=True, add_eos=True))
            while len(self._buffer) >= need:
                window = torch.tensor(self._buffer[:need], dtype=torch.int64)
                # the next window starts right after this one's inputs: its first token is this window's last label
                self._buffer = self._buffer[self.seq_len:]
                yield window

    def __iter__(self):
        batch = []
        for w in self._samples():
            batch.append(w)
            if len(batch) == self.batch_size:
                tok = torch.stack(batch)
                batch = []
                inputs = tok[:, : self.seq_len + self.extra].contiguous()
                labels = tok[:, 1:].contiguous()
                if self.pin:
                    inputs, labels = inputs.pin_memory(), labels.pin_memory()
                yield {"input": inputs}, labels

    def state_dict(self) -> dict[str, Any]:
        return {"sample_idx": self._sample_idx, "epoch": self._epoch, "buffer": list(self._buffer),
                "dp_world_size": self.dp_world_size}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        if not sd:
            return
        if int(sd.get("dp_world_size", self.dp_world_size)) != self.dp_world_size:
            raise ValueError("a text stream is sharded by data-parallel rank: resume with the same data-parallel "
                             f"degree ({sd['dp_world_size']}) or start the loader afresh")
        self._sample_idx, self._epoch = int(sd["sample_idx"]), int(sd.get("epoch", 0))
        self._buffer = list(sd.get("buffer", []))


def build_text_dataloader(cfg, *, tokenizer, training, dp_rank: int, dp_world_size: int) -> TextDataLoader:
    return TextDataLoader(dataset=cfg.dataset, dataset_path=cfg.dataset_path, tokenizer=tokenizer,
                          seq_len=training.seq_len, batch_size=training.local_batch_size, dp_rank=dp_rank,
                          dp_world_size=dp_world_size, extra_tokens=training.num_mtp_modules, infinite=cfg.infinite,
                          pin_memory=cfg.pin_memory)
