"""Variable-length ("TND") attention for Qwen3 recipes: packed documents attend within themselves only.

Parity: torchtitan_npu/models/qwen3/tnd_config.py:16-45 (`_enable_npu_varlen_attention`: swaps the attention core of
every layer and drops the upstream refusal of context parallelism for variable-length attention).
"""

from __future__ import annotations

from dataclasses import replace

__all__ = ["enable_varlen_attention"]


def enable_varlen_attention(model_ref):
    """Return a copy of a `ModelConfigRef` whose model is built with the variable-length attention core."""
    return replace(model_ref, overrides={**model_ref.overrides, "mask_type": "varlen"})
