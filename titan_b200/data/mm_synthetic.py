"""Multimodal batches: packed ``[<boi> <img>·n <eoi> caption <eos>]`` documents + patchified images.

A batch is ``({"input", "pixel_values", "grid_thw"}, labels)``:
* ``input``        ``[B, S]`` token ids; every image contributes ``h·w`` placeholder tokens;
* ``pixel_values`` ``[images, max_patches, C·p·p]`` flattened patches, zero-padded per image;
* ``grid_thw``     ``[images, max_patches, 3]`` (frame, row, column) of every patch, -1 on padding;
* ``labels``       next-token targets with image placeholders, padding and document starts masked (-100).

``dataset="synthetic"`` is a pure function of (seed, dp_rank, step): random captions and pixels of the right shapes,
for tests, dry runs and benchmarks without files.  Named datasets (image-caption pairs on disk) go through
`register_mm_dataset` with a sample iterator that yields ``(image [C, H, W] float tensor, caption token ids)``.

Parity: the upstream multimodal loader the reference's VLM recipe uses (torchtitan_npu/models/vlm/config_registry.py:
37-42: ``HuggingFaceMultiModalDataLoader(dataset="cc12m-test", max_patches_per_image=1024, max_images_per_batch=64)``).
"""

from __future__ import annotations

from collections.abc import Callable, Iterator
from typing import Any

import torch

__all__ = ["MultiModalDataLoader", "register_mm_dataset", "patchify", "build_mm_dataloader"]

IGNORE = -100
_DATASETS: dict[str, Callable[..., Iterator]] = {}


def register_mm_dataset(name: str, factory: Callable[..., Iterator]) -> None:
    """``factory(path, dp_rank, dp_world_size, seed) → iterator of (image [C,H,W], caption ids list[int])``."""
    _DATASETS[name] = factory


def patchify(image: torch.Tensor, patch: int, max_patches: int):
    """image [C, H, W] → (patches [h·w, C·p·p], grid [h·w, 3]); the image is cropped to whole patches and, if it has
    more than ``max_patches``, to the largest top-left block of rows that fits."""
    c, hh, ww = image.shape
    h, w = max(hh // patch, 1), max(ww // patch, 1)
    while h * w > max_patches:
        if h >= w:
            h -= 1
        else:
            w -= 1
    img = image[:, : h * patch, : w * patch]
    p = img.reshape(c, h, patch, w, patch).permute(1, 3, 0, 2, 4).reshape(h * w, c * patch * patch)
    rows = torch.arange(h).repeat_interleave(w)
    cols = torch.arange(w).repeat(h)
    return p, torch.stack([torch.zeros_like(rows), rows, cols], dim=-1)


class MultiModalDataLoader:
    def __init__(self, cfg, *, vocab_size: int, seq_len: int, batch_size: int, dp_rank: int, dp_world_size: int,
                 special_tokens, eos_id: int):
        self.cfg, self.vocab_size, self.seq_len, self.batch_size = cfg, vocab_size, seq_len, batch_size
        self.dp_rank, self.dp_world_size = dp_rank, dp_world_size
        self.sp, self.eos_id = special_tokens, eos_id
        self.patch_dim = cfg.n_channels * cfg.patch_size * cfg.patch_size
        self.pin = cfg.pin_memory and torch.cuda.is_available()
        self._step = 0
        self._source = None
        if cfg.dataset != "synthetic":
            if cfg.dataset not in _DATASETS:
                raise KeyError(f"unknown multimodal dataset {cfg.dataset!r}; registered: {sorted(_DATASETS)}")
            self._source = _DATASETS[cfg.dataset](cfg.dataset_path, dp_rank, dp_world_size, cfg.seed)
        reserved = {self.sp.img_id, self.sp.boi_id, self.sp.eoi_id, self.sp.pad_id, eos_id}
        self._text_hi = min(reserved | {vocab_size})  # captions draw ids below every reserved id

    # ---- one sample -------------------------------------------------------------------------------------------
    def _synthetic_sample(self, g: torch.Generator):
        side = int(self.cfg.max_patches_per_image ** 0.5)
        h = int(torch.randint(1, max(side, 1) + 1, (1,), generator=g))
        w = int(torch.randint(1, max(side, 1) + 1, (1,), generator=g))
        p = self.cfg.patch_size
        image = torch.rand(self.cfg.n_channels, h * p, w * p, generator=g)
        n = int(torch.randint(4, 33, (1,), generator=g))
        caption = torch.randint(3, max(self._text_hi, 4), (n,), generator=g).tolist()
        return image, caption

    def _batch(self, step: int):
        g = torch.Generator()
        g.manual_seed((self.cfg.seed * 1_000_003 + self.dp_rank) * 1_000_003 + step)
        S, B, L = self.seq_len, self.batch_size, self.cfg.max_patches_per_image
        tokens = torch.full((B, S + 1), self.sp.pad_id, dtype=torch.int64)
        pixels, grids = [], []
        for b in range(B):
            pos = 0
            while len(pixels) < self.cfg.max_images_per_batch:
                image, caption = next(self._source) if self._source is not None else self._synthetic_sample(g)
                patches, grid = patchify(image, self.cfg.patch_size, L)
                doc = [self.sp.boi_id] + [self.sp.img_id] * patches.shape[0] + [self.sp.eoi_id] + list(caption) \
                    + [self.eos_id]
                if pos + len(doc) > S + 1:
                    break
                tokens[b, pos: pos + len(doc)] = torch.tensor(doc)
                pos += len(doc)
                pad = L - patches.shape[0]
                pixels.append(torch.cat([patches, patches.new_zeros(pad, self.patch_dim)]))
                grids.append(torch.cat([grid, grid.new_full((pad, 3), -1)]))
        if not pixels:  # keep shapes non-empty: one fully padded image
            pixels.append(torch.zeros(L, self.patch_dim))
            grids.append(torch.full((L, 3), -1, dtype=torch.int64))
        inputs, labels = tokens[:, :-1].contiguous(), tokens[:, 1:].clone()
        for tid in (self.sp.img_id, self.sp.boi_id, self.sp.pad_id):
            labels[labels == tid] = IGNORE
        batch = {"input": inputs, "pixel_values": torch.stack(pixels), "grid_thw": torch.stack(grids)}
        if self.pin:
            batch = {k: v.pin_memory() for k, v in batch.items()}
            labels = labels.pin_memory()
        return batch, labels

    def __iter__(self):
        while True:
            try:
                batch = self._batch(self._step)
            except StopIteration:
                return
            self._step += 1
            yield batch

    def state_dict(self) -> dict[str, Any]:
        return {"step": self._step, "dp_world_size": self.dp_world_size}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        if state_dict:
            self._step = int(state_dict["step"])


def build_mm_dataloader(cfg, *, model_config, training, dp_rank: int, dp_world_size: int, tokenizer=None):
    from titan_b200.models.vlm.model import SpecialTokens

    sp = SpecialTokens(img_id=model_config.img_token_id, boi_id=model_config.boi_token_id,
                       eoi_id=model_config.eoi_token_id, pad_id=model_config.pad_token_id)
    eos = getattr(tokenizer, "eos_id", None)
    eos = model_config.eos_token_id if eos is None else eos
    if cfg.patch_size != model_config.encoder.patch_size or cfg.n_channels != model_config.encoder.n_channels:
        raise ValueError("dataloader patch_size / n_channels must match the vision encoder's")
    return MultiModalDataLoader(cfg, vocab_size=model_config.vocab_size, seq_len=training.seq_len,
                                batch_size=training.local_batch_size, dp_rank=dp_rank, dp_world_size=dp_world_size,
                                special_tokens=sp, eos_id=eos)
