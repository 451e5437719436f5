"""Context parallelism for DeepSeek-V4 attention (sliding window + compressed keys).

Every rank holds a contiguous slice of ``S_local`` tokens.  What a local query needs from other ranks is small:

* raw keys: only its causal window, i.e. the LAST ``W`` tokens of the previous rank.  Those ``W`` hidden states are sent
  point to point (rank r → r + 1) and prepended, so the projections, both compressors and the indexer simply run on
  ``W + S_local`` tokens with absolute positions.  ``W = max(window, ratio)`` rounded up to a multiple of ``ratio``: it
  also gives the ratio-4 compressor the previous block it overlaps with;
* compressed keys (one per ``ratio`` tokens) and indexer keys: the entries of the prepended region are dropped (their
  owner computes them), the local ones are all-gathered over the mesh and cut to the causal prefix
  ``[: (rank + 1) · S_local / ratio]``.

The attention core then sees ``S_local`` queries at global offset ``rank · S_local``, ``W + S_local`` raw keys and the
global compressed keys.  Backward: the window exchange returns the gradient of the prepended tokens to their owner
(point to point, added to the owner's last ``W`` tokens); the all-gather's backward is a reduce-scatter.

Parity: torchtitan_npu/distributed/context_parallel/compressor_attention_cp.py:72-306.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.device_mesh import DeviceMesh

from titan_b200.parallel.context_parallel.registry import register_cp_strategy
from titan_b200.parallel.context_parallel.sparse_attention_cp import _gather

__all__ = ["CompressorAttentionCP", "window_exchange"]


class _WindowExchange(torch.autograd.Function):
    """Prepend the previous rank's last ``window`` tokens (dim 1); rank 0 gets nothing prepended."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, window: int, group):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ctx.group, ctx.window, ctx.rank, ctx.world = group, window, rank, world
        reqs = []
        recv = None
        if rank > 0:
            recv = torch.empty_like(x[:, -window:])
            reqs.append(dist.irecv(recv, group=group, group_src=rank - 1))
        if rank + 1 < world:
            reqs.append(dist.isend(x[:, -window:].contiguous(), group=group, group_dst=rank + 1))
        for r in reqs:
            r.wait()
        return torch.cat([recv, x], dim=1) if recv is not None else x.clone()

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        rank, world, window, group = ctx.rank, ctx.world, ctx.window, ctx.group
        reqs = []
        back = None
        if rank > 0:
            reqs.append(dist.isend(g[:, :window].contiguous(), group=group, group_dst=rank - 1))
        if rank + 1 < world:
            back = torch.empty_like(g[:, :window])
            reqs.append(dist.irecv(back, group=group, group_src=rank + 1))
        for r in reqs:
            r.wait()
        own = g[:, window:] if rank > 0 else g
        if back is not None:
            own = own.clone()
            own[:, -window:] += back
        return own, None, None


def window_exchange(x: torch.Tensor, window: int, group) -> torch.Tensor:
    return _WindowExchange.apply(x, window, group)


class CompressorAttentionCP:
    def __init__(self, cp_mesh: DeviceMesh, compress_ratio: int, window_size: int):
        self.group = cp_mesh.get_group()
        self.cp, self.rank = cp_mesh.size(), cp_mesh.get_local_rank()
        self.ratio = max(int(compress_ratio), 1)
        w = max(int(window_size), self.ratio)
        self.window = (w + self.ratio - 1) // self.ratio * self.ratio

    def forward(self, attn: nn.Module, x: torch.Tensor, freqs_cis: torch.Tensor) -> torch.Tensor:
        B, s_local, _ = x.shape
        W, R, r = self.window, self.ratio, self.rank
        if s_local % R != 0 or s_local < W:
            raise ValueError(f"context-parallel slice of {s_local} tokens must be a multiple of the compression ratio "
                             f"{R} and at least the exchange window {W}")
        x_ext = window_exchange(x, W, self.group)
        lead = W if r > 0 else 0
        q_pos0 = r * s_local
        kv_pos0 = q_pos0 - lead
        positions = torch.arange(kv_pos0, q_pos0 + s_local, device=x.device).unsqueeze(0)
        q, kv, kvc, q_idx, k_idx, w = attn.pre_attention(x_ext, freqs_cis, positions)
        if lead:
            q = q[:, lead:]
            q_idx = q_idx[:, lead:] if q_idx is not None else None
            w = w[:, lead:] if w is not None else None
            kvc = kvc[:, lead // R:] if kvc is not None else None
            k_idx = k_idx[:, lead // R:] if k_idx is not None else None
        keep = (r + 1) * s_local // R
        if kvc is not None:
            kvc = _gather(kvc, 1, self.group, self.cp)[:, :keep]
        if k_idx is not None:
            k_idx = _gather(k_idx, 1, self.group, self.cp)[:, :keep]
        o = attn.inner_attention(q.contiguous(), kv, kvc, q_idx, k_idx, w, q_pos0=q_pos0, kv_pos0=kv_pos0)
        return attn.post_attention(o, freqs_cis, positions[:, lead:])

    def apply(self, attn: nn.Module) -> nn.Module:
        attn.cp = self
        attn._cp_strategy = "compressor_window_exchange"
        return attn


def _is_v4_attention(mod: nn.Module) -> bool:
    return hasattr(mod, "pre_attention") and hasattr(mod, "inner_attention") and \
        hasattr(mod.inner_attention, "compress_ratio")


def _apply(mod: nn.Module, mesh: DeviceMesh) -> nn.Module:
    inner = mod.inner_attention
    return CompressorAttentionCP(mesh, inner.compress_ratio, inner.window).apply(mod)


register_cp_strategy("compressor_window_exchange", _is_v4_attention, _apply, first=True)
