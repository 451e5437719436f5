"""Synthetic token loader: uniform-random ids from a fixed seed.

Each data-parallel rank draws from its own generator stream (seed + dp_rank), so
a run is reproducible and ranks see different data.  Batches are produced in
pinned host memory so the trainer's H2D copy is asynchronous.  The loader is
stateful (step counter) and resumes exactly from a checkpoint.

The reference's own tiny test corpus is a missing large blob
(tests/assets/c4_test, `.MISSING_LARGE_BLOBS`), so random ids of the named shape
are the hardware-free data source here.
"""

from __future__ import annotations

from typing import Any

import torch
from torch.distributed.checkpoint.stateful import Stateful

__all__ = ["SyntheticDataLoader", "build_dataloader"]


class SyntheticDataLoader(Stateful):
    def __init__(self, *, vocab_size: int, seq_len: int, batch_size: int, dp_rank: int = 0, dp_world_size: int = 1,
                 seed: int = 0, pin_memory: bool = True, extra_tokens: int = 0, infinite: bool = True,
                 documents_per_row: int = 0, global_stream: bool = False):
        self.vocab_size = vocab_size
        self.seq_len = seq_len
        self.batch_size = batch_size
        self.dp_rank = dp_rank
        self.dp_world_size = dp_world_size
        self.seed = seed
        self.extra_tokens = extra_tokens  # MTP needs `num_mtp` more label tokens
        self.pin_memory = pin_memory and torch.cuda.is_available()
        self.documents_per_row = documents_per_row  # > 0: rows are packed documents and carry `positions`
        # one stream for the whole job: every step draws the GLOBAL batch and each data-parallel rank keeps its rows,
        # so N ranks x batch b see exactly the rows of 1 rank x batch N*b (parallel runs become comparable)
        self.global_stream = global_stream
        self._step = 0

    def _batch(self, step: int):
        g = torch.Generator()
        n = self.seq_len + 1 + self.extra_tokens
        if self.global_stream:
            g.manual_seed(self.seed * 1_000_003 * 1_000_003 + step)
            tok = torch.randint(0, self.vocab_size, (self.batch_size * self.dp_world_size, n), generator=g,
                                dtype=torch.int64)
            tok = tok[self.dp_rank * self.batch_size: (self.dp_rank + 1) * self.batch_size]
        else:
            g.manual_seed((self.seed * 1_000_003 + self.dp_rank) * 1_000_003 + step)
            tok = torch.randint(0, self.vocab_size, (self.batch_size, n), generator=g, dtype=torch.int64)
        # with MTP the model gets the look-ahead tokens too: depth k embeds inputs[:, k : k + seq_len]
        inputs = tok[:, : self.seq_len + self.extra_tokens].contiguous()
        labels = tok[:, 1:].contiguous()
        batch = {"input": inputs}
        if self.documents_per_row > 0:
            # random document boundaries: position inside the document for each of the seq_len main tokens
            width = self.seq_len
            cuts = torch.rand(self.batch_size, width, generator=g) < (self.documents_per_row - 1) / max(width, 1)
            cuts[:, 0] = True
            idx = torch.arange(width).expand(self.batch_size, width)
            start = torch.where(cuts, idx, torch.zeros_like(idx)).cummax(dim=1).values
            batch["positions"] = (idx - start).contiguous()
        if self.pin_memory:
            batch = {k: v.pin_memory() for k, v in batch.items()}
            labels = labels.pin_memory()
        return batch, labels

    def __iter__(self):
        while True:
            batch = self._batch(self._step)
            self._step += 1
            yield batch

    def state_dict(self) -> dict[str, Any]:
        return {"step": self._step, "dp_world_size": self.dp_world_size}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        if not state_dict:
            return
        # the stream is a pure function of (seed, dp_rank, step): a different data-parallel degree on
        # resume continues at the same step with its own rank streams
        self._step = int(state_dict["step"])


def build_dataloader(cfg, *, model_config, training, dp_rank: int, dp_world_size: int, tokenizer=None):
    """Build the loader named by the `dataloader` section of the trainer config."""
    from titan_b200.config.configs import ChatDataLoaderConfig, SyntheticDataLoaderConfig, TextDataLoaderConfig

    extra = training.num_mtp_modules
    if isinstance(cfg, SyntheticDataLoaderConfig):
        return SyntheticDataLoader(
            vocab_size=cfg.vocab_size or model_config.vocab_size, seq_len=training.seq_len,
            batch_size=training.local_batch_size, dp_rank=dp_rank, dp_world_size=dp_world_size, seed=cfg.seed,
            pin_memory=cfg.pin_memory, extra_tokens=extra, infinite=cfg.infinite,
            documents_per_row=cfg.documents_per_row, global_stream=cfg.global_stream,
        )
    if isinstance(cfg, TextDataLoaderConfig):
        from titan_b200.data.text_datasets import build_text_dataloader

        return build_text_dataloader(cfg, tokenizer=tokenizer, training=training, dp_rank=dp_rank,
                                     dp_world_size=dp_world_size)
    if isinstance(cfg, ChatDataLoaderConfig):
        from titan_b200.data.chat_dataset import build_chat_dataloader

        return build_chat_dataloader(cfg, tokenizer=tokenizer, training=training, dp_rank=dp_rank,
                                     dp_world_size=dp_world_size)
    from titan_b200.config.configs import MultiModalDataLoaderConfig

    if isinstance(cfg, MultiModalDataLoaderConfig):
        from titan_b200.data.mm_synthetic import build_mm_dataloader

        return build_mm_dataloader(cfg, model_config=model_config, training=training, dp_rank=dp_rank,
                                   dp_world_size=dp_world_size, tokenizer=tokenizer)
    raise TypeError(f"unknown dataloader config {type(cfg).__name__}")
