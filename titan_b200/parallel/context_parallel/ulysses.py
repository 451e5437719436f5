"""Ulysses context parallelism: head ↔ sequence all-to-all around a full-sequence attention core.

Before attention q, k, v ``[B, H, S/cp, D]`` are exchanged so every rank holds ``H/cp`` heads over the
whole sequence; the plain causal kernel then runs unchanged; the output is exchanged back.  Every
rank does the same amount of attention work, so no load balancing (and no sequence reordering) is
needed.  Requires ``H % cp == 0`` (and ``H_kv % cp == 0`` under GQA).

`AllToAll` is the autograd primitive: chunk the scatter dim → equal-split all-to-all → concatenate on
the gather dim; backward swaps the two dims.

Parity: torchtitan_npu/distributed/context_parallel/ulysses_cp.py:28-115.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.device_mesh import DeviceMesh

from titan_b200.parallel.context_parallel.registry import register_cp_strategy
from titan_b200.parallel.fake_pg import is_fake_process_group

__all__ = ["AllToAll", "UlyssesCP", "all_to_all_4d"]


def _a2a(x: torch.Tensor, scatter_dim: int, gather_dim: int, group) -> torch.Tensor:
    ws = dist.get_world_size(group)
    if ws == 1:
        return x
    if x.shape[scatter_dim] % ws != 0:
        raise ValueError(f"dim {scatter_dim} of size {x.shape[scatter_dim]} is not divisible by cp={ws}")
    # [ws, ...chunk...] with the peer index leading so one equal-split all-to-all moves every chunk
    chunks = torch.stack(torch.chunk(x, ws, dim=scatter_dim), dim=0).contiguous()
    out = torch.empty_like(chunks)
    if is_fake_process_group(group):
        out = chunks
    else:
        dist.all_to_all_single(out, chunks, group=group)
    gd = gather_dim % x.dim()
    return torch.cat(list(out.unbind(0)), dim=gd)


class AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scatter_dim, gather_dim, group):
        ctx.scatter_dim, ctx.gather_dim, ctx.group = scatter_dim, gather_dim, group
        return _a2a(x, scatter_dim, gather_dim, group)

    @staticmethod
    def backward(ctx, g):
        return _a2a(g.contiguous(), ctx.gather_dim, ctx.scatter_dim, ctx.group), None, None, None


def all_to_all_4d(x, scatter_dim, gather_dim, group):
    return AllToAll.apply(x, scatter_dim, gather_dim, group)


class UlyssesCP:
    """Hooks for attention cores called as ``core(q, k, v, ...)`` on ``[B, H, S, D]`` tensors."""

    head_dim_index = 1
    seq_dim_index = 2

    def __init__(self, cp_mesh: DeviceMesh):
        self.group = cp_mesh.get_group()
        self.cp = cp_mesh.size()

    def pre(self, module, args, kwargs):
        q, k, v, *rest = args
        h, s = self.head_dim_index, self.seq_dim_index
        for name, t in (("q", q), ("k", k), ("v", v)):
            if t.shape[h] % self.cp != 0:
                raise ValueError(f"Ulysses CP: {name} has {t.shape[h]} heads, not divisible by cp={self.cp}")
        q = all_to_all_4d(q, h, s, self.group)
        k = all_to_all_4d(k, h, s, self.group)
        v = all_to_all_4d(v, h, s, self.group)
        return (q, k, v, *rest), kwargs

    def post(self, module, args, kwargs, out):
        return all_to_all_4d(out, self.seq_dim_index, self.head_dim_index, self.group)

    def apply(self, module: nn.Module) -> nn.Module:
        module.register_forward_pre_hook(self.pre, with_kwargs=True)
        module.register_forward_hook(self.post, with_kwargs=True)
        module._cp_strategy = "ulysses"
        return module


def _is_sdpa_core(mod: nn.Module) -> bool:
    from titan_b200.models.common.layers import ScaledDotProductAttention

    return isinstance(mod, ScaledDotProductAttention) or getattr(mod, "cp_layout", None) == "bhsd"


register_cp_strategy("ulysses", _is_sdpa_core, lambda m, mesh: UlyssesCP(mesh).apply(m))
