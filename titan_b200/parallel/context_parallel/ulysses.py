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


# ------------------------------------------------------------------------------------------------------------------
# Fused form: the two exchanges disappear into the projections next to them.  `wq / wk / wv` become GEMMs whose
# epilogue stores each head slice into the owner's receive buffer; `wo` becomes a GEMM that pulls the head slices of
# its rows from the peers while it runs (ops/ulysses_fused.py).  RoPE and the per-head q/k norms act per position and
# per head, so they commute with the exchange and run afterwards on (all positions, local heads).
def _gather_positions(positions: torch.Tensor | None, group, cp: int):
    if positions is None or cp == 1:
        return positions
    local = positions.contiguous().view(-1, positions.shape[-1])  # [rows, S_local]
    out = torch.empty((cp * local.shape[0], local.shape[1]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local, group=group)
    full = out.view(cp, local.shape[0], local.shape[1]).transpose(0, 1).reshape(local.shape[0], -1)
    return full.view(*positions.shape[:-1], cp * positions.shape[-1])


def apply_fused_ulysses(attn: nn.Module, cp_mesh: DeviceMesh, rope_fn) -> nn.Module:
    """Replace ``attn.forward`` (an attention block with bias-free ``wq, wk, wv, wo`` projections, ``head_dim``, an
    optional ``q_norm / k_norm`` pair and an ``inner_attention`` core taking ``[B, H, S, D]``) by the fused form.
    ``rope_fn(xq, xk, rope_cache, positions)`` is the model's rotary embedding on ``[B, S, H, D]``."""
    from titan_b200.ops.ulysses_fused import all_to_all_proj, proj_all_to_all

    group, cp = cp_mesh.get_group(), cp_mesh.size()
    for name in ("wq", "wk", "wv", "wo"):
        lin = getattr(attn, name)
        if getattr(lin, "bias", None) is not None:
            raise NotImplementedError(f"fused Ulysses projections need bias-free linears ({name} has a bias)")
    hd = attn.head_dim

    def forward(x, rope_cache, attention_masks=None, positions=None):
        bs, s_loc, dim = x.shape
        x2 = x.reshape(bs * s_loc, dim)

        def w(lin):
            t = lin.weight
            if hasattr(t, "to_local"):
                raise NotImplementedError("fused Ulysses projections do not compose with tensor parallelism")
            return t.to(x2.dtype)

        q = proj_all_to_all(x2, w(attn.wq), s_loc, group).view(bs, cp * s_loc, -1, hd)
        k = proj_all_to_all(x2, w(attn.wk), s_loc, group).view(bs, cp * s_loc, -1, hd)
        v = proj_all_to_all(x2, w(attn.wv), s_loc, group).view(bs, cp * s_loc, -1, hd)
        if getattr(attn, "q_norm", None) is not None:
            q, k = attn.q_norm(q), attn.k_norm(k)
        q, k = rope_fn(q, k, rope_cache, _gather_positions(positions, group, cp))
        out = attn.inner_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=attention_masks)
        o = out.transpose(1, 2).reshape(bs * cp * s_loc, -1)
        return all_to_all_proj(o, w(attn.wo), s_loc, group).view(bs, s_loc, dim)

    attn.forward = forward
    attn._cp_strategy = "ulysses_fused"
    return attn
