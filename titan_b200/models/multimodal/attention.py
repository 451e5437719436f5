"""Library attention with a dense boolean mask ``(B, S, S)`` (True = may attend); tensors in ``(B, H, S, D)``.

Parity: `DenseMaskSDPA` (torchtitan_npu/models/multimodal/attention.py:10-60).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from titan_b200.protocols.module import Module

__all__ = ["DenseMaskSDPA"]


class DenseMaskSDPA(Module):
    needs_attention_masks = True  # the trainer asks the model for masks when a core says so

    def __init__(self):
        super().__init__()

    def forward(self, q, k, v, *, scale: float | None = None, attn_mask: torch.Tensor | None = None):
        if attn_mask is not None and attn_mask.dim() == 3:
            attn_mask = attn_mask[:, None, :, :]
        gqa = q.shape[1] != k.shape[1]
        if attn_mask is None:
            return F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=gqa)
        return F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask.to(q.device), scale=scale, enable_gqa=gqa)
