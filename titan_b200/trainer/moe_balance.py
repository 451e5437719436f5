"""Auxiliary-loss-free MoE load balancing, run as an optimizer pre-step hook.

Per MoE layer the number of tokens routed to each expert since the last step is summed over all
data/context-parallel ranks (one all-reduce of a ``[L_moe, E]`` matrix over the ``loss`` mesh), then
``expert_bias += coeff * sign(mean - tokens)`` with the update re-centred to zero mean.  Layers
without an ``expert_bias`` buffer (hash-routed layers) are tolerated.  Under non-reentrant
activation checkpointing the forward runs twice, so counts are halved.

Parity: torchtitan_npu/patches/torchtitan/optimizer.py:42-124.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

__all__ = ["register_moe_load_balancing_hook", "update_expert_bias"]


def _blocks(part: nn.Module):
    layers = getattr(part, "layers", None)
    if layers is None:
        return []
    return [b for b in layers.values() if b is not None]


def _unwrap(block: nn.Module):
    """(inner block, was it wrapped for recomputation?)"""
    inner = getattr(block, "_checkpoint_wrapped_module", None)
    return (inner, True) if inner is not None else (block, False)


def update_expert_bias(model_parts: list[nn.Module], parallel_dims) -> None:
    rows, moes = [], []
    for part in model_parts:
        for blk in _blocks(part):
            inner, recompute = _unwrap(blk)
            if not getattr(inner, "moe_enabled", False):
                continue
            moe = inner.moe
            if moe.load_balance_coeff is None:
                return
            t = moe.tokens_per_expert
            rows.append(t // 2 if recompute else t)
            moes.append(moe)
    if not rows:
        return
    mat = torch.vstack(rows)
    # layers whose tokens stay sequence-sharded over tensor-parallel ranks count per-rank slices
    slice_group = next((g for g in (getattr(m, "counts_group", None) for m in moes) if g is not None), None)
    if slice_group is not None and dist.is_initialized():
        dist.all_reduce(mat, group=slice_group, op=dist.ReduceOp.SUM)
    loss_mesh = parallel_dims.get_optional_mesh("loss") if (parallel_dims is not None and dist.is_initialized()) else None
    if loss_mesh is not None:
        dist.all_reduce(mat, group=loss_mesh.get_group(), op=dist.ReduceOp.SUM)
    with torch.no_grad():
        for i, moe in enumerate(moes):
            tokens = mat[i].float()
            delta = moe.load_balance_coeff * torch.sign(tokens.mean() - tokens)
            delta = delta - delta.mean()
            bias = getattr(moe, "expert_bias", None)
            if bias is not None:
                bias.add_(delta)
            moe.tokens_per_expert.zero_()


def register_moe_load_balancing_hook(optimizers, model_parts: list[nn.Module], parallel_dims) -> None:
    enabled = False
    for part in model_parts:
        for blk in _blocks(part):
            inner, _ = _unwrap(blk)
            if getattr(inner, "moe_enabled", False):
                enabled = bool(inner.moe.load_balance_coeff)
                break
        if enabled:
            break
    if enabled:
        optimizers.register_step_pre_hook(lambda *a, **k: update_expert_bias(model_parts, parallel_dims))
