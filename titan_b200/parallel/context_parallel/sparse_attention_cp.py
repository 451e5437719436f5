"""Context parallelism for DeepSeek sparse attention (DSA): all-gather the shared KV latent and indexer keys.

Queries stay sequence-local.  The single-head KV latent ``k, v [B, 1, S/cp, D]`` and the indexer keys
``k_indexer [B, S/cp, 1, 128]`` are all-gathered over the ``cp`` mesh (small: one head), then cut to the
causal prefix ``[: (rank + 1) · S_local]`` so rank r attends to everything up to its own block; the
attention core treats the local queries as the tail of that key range.  Backward of the gather is a
reduce-scatter.  Work grows with the rank; no balancing is applied
because top-k selection bounds the attention cost and the indexer is cheap.

Parity: torchtitan_npu/distributed/context_parallel/sparse_attention_cp.py:30-90.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh

from titan_b200.parallel.context_parallel.registry import register_cp_strategy
from titan_b200.parallel.fake_pg import is_fake_process_group

__all__ = ["SparseAttentionCP"]


def _gather(x: torch.Tensor, dim: int, group, world: int) -> torch.Tensor:
    if world == 1:
        return x
    if is_fake_process_group(group):
        return torch.cat([x] * world, dim=dim)
    return _AllGatherDim.apply(x, dim, group, world)


class _AllGatherDim(torch.autograd.Function):
    """All-gather along ``dim``; the backward is the matching reduce-scatter (sum) of the gathered gradient."""

    @staticmethod
    def forward(ctx, x, dim, group, world):
        ctx.dim, ctx.group, ctx.world = dim, group, world
        xt = x.movedim(dim, 0).contiguous()
        out = xt.new_empty((world * xt.shape[0], *xt.shape[1:]))
        dist.all_gather_into_tensor(out, xt, group=group)
        return out.movedim(0, dim)

    @staticmethod
    def backward(ctx, g):
        gt = g.movedim(ctx.dim, 0).contiguous()
        out = gt.new_empty((gt.shape[0] // ctx.world, *gt.shape[1:]))
        dist.reduce_scatter_tensor(out, gt, op=dist.ReduceOp.SUM, group=ctx.group)
        return out.movedim(0, ctx.dim), None, None, None


class SparseAttentionCP:
    def __init__(self, cp_mesh: DeviceMesh):
        self.group = cp_mesh.get_group()
        self.cp, self.rank = cp_mesh.size(), cp_mesh.get_local_rank()

    def pre(self, module, args, kwargs):
        q, k, v, *rest = args
        s_local = k.shape[2]
        keep = (self.rank + 1) * s_local
        k = _gather(k, 2, self.group, self.cp)[:, :, :keep]
        v = _gather(v, 2, self.group, self.cp)[:, :, :keep]
        kw = dict(kwargs)
        if kw.get("k_indexer") is not None:
            kw["k_indexer"] = _gather(kw["k_indexer"], 1, self.group, self.cp)[:, :keep]
        if kw.get("attn_mask") is not None:
            raise NotImplementedError("DSA CP builds its own causal mask; custom masks are not supported")
        return (q, k, v, *rest), kw

    def apply(self, module: nn.Module) -> nn.Module:
        module.register_forward_pre_hook(self.pre, with_kwargs=True)
        module._cp_strategy = "dsa_allgather"
        return module


def _is_dsa_core(mod: nn.Module) -> bool:
    return getattr(mod, "cp_layout", None) == "dsa" or type(mod).__name__ in ("DSASparseAttention", "FusedDSAttention")


register_cp_strategy("dsa_allgather", _is_dsa_core, lambda m, mesh: SparseAttentionCP(mesh).apply(m), first=True)
