"""Variable-length ("TND") attention core for packed documents.

The trainer hands a batch of packed sequences with position ids that restart at every document.  `VarlenMetadata`
turns them into cumulative document boundaries once per step; `VarlenAttention` then runs causal attention per
document.  On a B200 (bf16, head dim 128, sequence a multiple of 128, documents up to `KERNEL_MAX_DOCUMENT` tokens)
that is ONE launch of the tcgen05 flash kernels with the per-token document start as the mask
(`titan_b200.ops.flash_attention`, forward and backward); elsewhere one library SDPA call per document, which sees a plain causal problem and needs no ``S × S`` mask.  Under Ulysses context
parallelism the core sees the full sequence with a slice of the heads, so the same metadata applies unchanged.

Parity: `NPUVarlenAttention` (torchtitan_npu/models/common/npu_varlen_attention.py) used by the Qwen3 TND recipe
(models/qwen3/tnd_config.py:20-45).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from titan_b200.protocols.module import Module

__all__ = ["VarlenMetadata", "VarlenAttention", "build_varlen_metadata"]

# Packed batches of short documents go through ONE launch of the tcgen05 flash kernels (document masks inside); with
# long documents the per-document library calls win (fewer launches to save, and the library's dense kernel is faster
# per FLOP), so rows whose longest document exceeds this many tokens take the per-document path.
KERNEL_MAX_DOCUMENT = 2048


@dataclass
class VarlenMetadata:
    cu_seqlens: list[list[int]]  # per batch row: document boundaries [0, ..., S]
    max_seqlen: int

    def to(self, *args, **kwargs):  # moves with the batch like a tensor would
        return self

    def seq_start(self, device) -> torch.Tensor:
        """[B, S] int32: the position of the first token of each token's document (built once per step)."""
        cached = self.__dict__.get("_seq_start")
        if cached is None or cached.device != torch.device(device):
            rows = []
            for bounds in self.cu_seqlens:
                b = torch.tensor(bounds, dtype=torch.int64)
                rows.append(torch.repeat_interleave(b[:-1], b[1:] - b[:-1]))
            cached = torch.stack(rows).to(torch.int32).to(device)
            self.__dict__["_seq_start"] = cached
        return cached


def build_varlen_metadata(positions: torch.Tensor) -> VarlenMetadata:
    """positions [B, S] (or [S]) restart at 0 at every document start."""
    if positions.dim() == 1:
        positions = positions.unsqueeze(0)
    pos = positions.detach().cpu()
    out, longest = [], 0
    s = pos.shape[1]
    for row in pos:
        starts = (row == 0).nonzero().flatten().tolist()
        if not starts or starts[0] != 0:
            starts = [0] + starts
        bounds = starts + [s]
        longest = max(longest, max(b - a for a, b in zip(bounds[:-1], bounds[1:])))
        out.append(bounds)
    return VarlenMetadata(out, longest)


class VarlenAttention(Module):
    """q, k, v: [B, H, S, D] → [B, H, S, D]; ``attn_mask`` carries a `VarlenMetadata` (None = one document)."""

    def __init__(self):
        super().__init__()

    def forward(self, q, k, v, *, scale: float | None = None, attn_mask=None):
        gqa = q.shape[1] != k.shape[1]
        if attn_mask is None:
            return F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=gqa)
        if not isinstance(attn_mask, VarlenMetadata):
            return F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, scale=scale, enable_gqa=gqa)
        from titan_b200.ops.flash_attention import flash_attention, flash_attention_supported

        if (q.is_cuda and flash_attention_supported(q, k) and v.shape[-1] == q.shape[-1]
                and attn_mask.max_seqlen <= KERNEL_MAX_DOCUMENT):
            return flash_attention(q, k, v, scale=scale, seq_start=attn_mask.seq_start(q.device))
        rows = []
        for b, bounds in enumerate(attn_mask.cu_seqlens):
            docs = []
            for a, e in zip(bounds[:-1], bounds[1:]):
                docs.append(F.scaled_dot_product_attention(q[b:b + 1, :, a:e], k[b:b + 1, :, a:e], v[b:b + 1, :, a:e],
                                                           is_causal=True, scale=scale, enable_gqa=gqa))
            rows.append(torch.cat(docs, dim=2))
        return torch.cat(rows, dim=0)
