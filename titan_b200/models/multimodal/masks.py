"""Dense boolean attention masks for multimodal models (True = the query may attend to the key).

* text: causal within a packed document (documents end with EOS);
* vision encoder: over valid patches only (causal or full); image batches are zero-padded to a common patch count and
  padded patches carry the coordinate ``PADDED_PATCH_COORDINATE``.  A fully masked softmax row yields NaN in the library
  attention, so padded query rows may keep their diagonal element: their outputs are dropped afterwards.

Parity: torchtitan_npu/models/multimodal/masks.py:10-98.
"""

from __future__ import annotations

import torch

__all__ = ["PADDED_PATCH_COORDINATE", "build_causal_mask", "build_document_ids", "build_text_document_causal_mask",
           "build_valid_patch_mask", "build_encoder_causal_mask", "build_encoder_full_mask"]

PADDED_PATCH_COORDINATE = -1


def build_causal_mask(seq_len: int, device=None) -> torch.Tensor:
    pos = torch.arange(seq_len, device=device)
    return pos[:, None] >= pos[None, :]


def build_document_ids(tokens: torch.Tensor, eos_id: int) -> torch.Tensor:
    """Document index of every token; an EOS token belongs to the document it closes."""
    if tokens.dim() != 2:
        raise ValueError("tokens must have shape (batch, seq_len)")
    eos = tokens == eos_id
    ids = eos.cumsum(dim=1)
    return ids - eos.to(ids.dtype)


def build_text_document_causal_mask(tokens: torch.Tensor, eos_id: int) -> torch.Tensor:
    if tokens.dim() != 2:
        raise ValueError("tokens must have shape (batch, seq_len)")
    b, s = tokens.shape
    doc = build_document_ids(tokens, eos_id)
    return build_causal_mask(s, tokens.device).expand(b, s, s) & (doc[:, :, None] == doc[:, None, :])


def build_valid_patch_mask(grid_hw: torch.Tensor) -> torch.Tensor:
    """grid_hw ``(images, patches, 2)`` → ``(images, patches)``: True where both coordinates are real."""
    if grid_hw.dim() != 3 or grid_hw.shape[-1] != 2:
        raise ValueError("grid_hw must have shape (batch, seq_len, 2)")
    return (grid_hw != PADDED_PATCH_COORDINATE).all(dim=-1)


def _keep_padding_diagonal(mask: torch.Tensor, valid: torch.Tensor) -> torch.Tensor:
    eye = torch.eye(valid.shape[1], dtype=torch.bool, device=valid.device)
    return mask | (~valid[:, :, None] & eye)


def build_encoder_causal_mask(valid_tokens: torch.Tensor, *, allow_padding_self_attention: bool = True):
    if valid_tokens.dim() != 2:
        raise ValueError("valid_tokens must have shape (batch, seq_len)")
    valid = valid_tokens.to(torch.bool)
    b, s = valid.shape
    mask = build_causal_mask(s, valid.device).expand(b, s, s) & (valid[:, :, None] & valid[:, None, :])
    return _keep_padding_diagonal(mask, valid) if allow_padding_self_attention else mask


def build_encoder_full_mask(valid_tokens: torch.Tensor, *, allow_padding_self_attention: bool = True):
    if valid_tokens.dim() != 2:
        raise ValueError("valid_tokens must have shape (batch, seq_len)")
    valid = valid_tokens.to(torch.bool)
    mask = valid[:, :, None] & valid[:, None, :]
    return _keep_padding_diagonal(mask, valid) if allow_padding_self_attention else mask
