"""Ulysses context parallelism for packed variable-length ("TND") attention.

`VarlenAttention` is called as ``core(q, k, v, attn_mask=VarlenMetadata)`` on ``[B, H, S, D]`` tensors, the layout
`UlyssesCP` exchanges: after the head <-> sequence all-to-all a rank holds ``H / cp`` heads over the FULL packed
sequence, so the document boundaries that the trainer derived from the full sequence apply as they are.  Two
pieces make that work:

* a strategy entry that accepts `VarlenAttention` (placed before the generic SDPA entry so that a model mixing both
  cores is told which hook it got), and
* a mask handler that hands `VarlenMetadata` through untouched: the generic path would slice a mask to the
  rank's sequence shard, which for document boundaries would be wrong on every rank but the first.

Parity: `NPUVarlenUlyssesCP` and its mask handler
(torchtitan_npu/distributed/context_parallel/npu_varlen_cp.py:30-79).
"""

from __future__ import annotations

import torch.nn as nn

from titan_b200.parallel.context_parallel.registry import register_cp_mask_handler, register_cp_strategy
from titan_b200.parallel.context_parallel.ulysses import UlyssesCP

__all__ = ["VarlenUlyssesCP", "varlen_mask_handler"]


class VarlenUlyssesCP(UlyssesCP):
    def apply(self, module: nn.Module) -> nn.Module:
        super().apply(module)
        module._cp_strategy = "ulysses_varlen"
        return module


def _is_varlen_core(mod: nn.Module) -> bool:
    from titan_b200.models.common.varlen_attention import VarlenAttention

    return isinstance(mod, VarlenAttention)


def varlen_mask_handler(masks, cp_mesh):
    from titan_b200.models.common.varlen_attention import VarlenMetadata

    return masks if isinstance(masks, VarlenMetadata) else None


register_cp_strategy("ulysses_varlen", _is_varlen_core, lambda m, mesh: VarlenUlyssesCP(mesh).apply(m), first=True)
register_cp_mask_handler(varlen_mask_handler)
