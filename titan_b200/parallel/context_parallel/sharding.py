"""Sequence sharding of a batch for context parallelism, MTP-aware.

Each CP rank keeps a contiguous slice of the sequence (no head-tail / round-robin reordering:
Ulysses, DSA and compressor CP all rebuild or assume contiguous order, so a balancer would break
causality).  With multi-token prediction the labels carry ``num_mtp`` extra shifted tokens: rank r
keeps labels ``[r·S_loc, (r+1)·S_loc + num_mtp)`` so every local position still sees all of its
targets; positions are sharded consistently.

Parity: torchtitan_npu/patches/distributed/mtp_context_parallel.py:32-110,
patches/distributed/cp_shard_mask.py:26-59 (custom masks go to handlers; balancers are rejected).
"""

from __future__ import annotations

import torch

from titan_b200.parallel.context_parallel.registry import adjust_cp_mask

__all__ = ["cp_shard", "prepare_context_parallel_input"]


def cp_shard(t: torch.Tensor, cp_rank: int, cp_size: int, seq_dim: int = 1, extra: int = 0) -> torch.Tensor:
    total = t.shape[seq_dim] - extra
    if total % cp_size != 0:
        raise ValueError(f"sequence length {total} is not divisible by cp={cp_size}")
    loc = total // cp_size
    return t.narrow(seq_dim, cp_rank * loc, loc + extra)


def prepare_context_parallel_input(inputs, labels, extra_kwargs, *, cp_mesh, device, num_mtp_modules: int = 0,
                                   load_balancer: str | None = None):
    if load_balancer not in (None, "none", ""):
        raise NotImplementedError(
            f"context_parallel_load_balancer={load_balancer!r}: sequence reordering breaks the contiguous causal "
            "layout that Ulysses / DSA / compressor CP rely on; set it to None")
    cp, r = cp_mesh.size(), cp_mesh.get_local_rank()
    seq = inputs.shape[1]
    positions = extra_kwargs.get("positions")
    if positions is None:
        positions = torch.arange(seq, device=inputs.device, dtype=torch.int64).unsqueeze(0)
    inputs = cp_shard(inputs, r, cp).contiguous()
    labels = cp_shard(labels, r, cp, extra=num_mtp_modules).contiguous()
    out_kwargs = dict(extra_kwargs)
    out_kwargs["positions"] = cp_shard(positions, r, cp).contiguous()
    if out_kwargs.get("attention_masks") is not None:
        out_kwargs["attention_masks"] = adjust_cp_mask(out_kwargs["attention_masks"], cp_mesh)
    return inputs, labels, out_kwargs
