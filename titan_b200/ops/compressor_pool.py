"""Gated softmax pooling of the DeepSeek-V4 KV compressor: ``Σ_slot softmax(score + ape) · kv`` per block of ``ratio``
tokens (ratio 4 pools 2·ratio overlapping candidates), fp32, with a CUDA kernel pair (`csrc/elementwise/
compressor_pool.cu`) and the PyTorch form as reference and CPU path.

Parity: the pooling inside ``Compressor._forward_bsnd`` / ``_forward_tnd`` of the reference's DeepSeek-V4 model
(torchtitan_npu/models/deepseek_v4/model.py) — the op its `compressor` kernel slot stands for.
"""

from __future__ import annotations

import ctypes

import torch

from titan_b200.ops import _lib

__all__ = ["compressor_pool", "compressor_pool_ref"]

_DECLARED = False


def _overlap(t: torch.Tensor, d: int, fill: float) -> torch.Tensor:
    """[B, C, r, 2d] → [B, C, 2r, d]: slots r.. = this block's second half, slots ..r = previous block's first half."""
    B, C, r, _ = t.shape
    out = t.new_full((B, C, 2 * r, d), fill)
    out[:, :, r:] = t[..., d:]
    out[:, 1:, :r] = t[:, :-1, :, :d]
    return out


def compressor_pool_ref(kv: torch.Tensor, score: torch.Tensor, ape: torch.Tensor, ratio: int, head_dim: int,
                        overlap: bool) -> torch.Tensor:
    """kv, score [B, S, width] → [B, S / ratio, head_dim] (PyTorch, any device)."""
    kv = kv.unflatten(1, (-1, ratio))
    score = score.unflatten(1, (-1, ratio)) + ape
    if overlap:
        kv, score = _overlap(kv, head_dim, 0.0), _overlap(score, head_dim, float("-inf"))
    return (kv * score.softmax(dim=2)).sum(dim=2)


def _declare():
    global _DECLARED
    if not _DECLARED:
        P, I = ctypes.c_void_p, ctypes.c_int
        _lib.declare("tb_compressor_pool_fwd", [P, P, P, P, P, I, I, I, I, I, P])
        _lib.declare("tb_compressor_pool_bwd", [P, P, P, P, P, P, P, P, I, I, I, I, I, P])
        _DECLARED = True


class _PoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, kv, score, ape, ratio, head_dim, overlap):
        _declare()
        kv, score, ape = kv.contiguous(), score.contiguous(), ape.contiguous()
        B, S, _ = kv.shape
        out = torch.empty(B, S // ratio, head_dim, dtype=torch.float32, device=kv.device)
        lse = torch.empty_like(out)
        rc = _lib.lib().tb_compressor_pool_fwd(kv.data_ptr(), score.data_ptr(), ape.data_ptr(), out.data_ptr(),
                                               lse.data_ptr(), B, S, ratio, head_dim, int(overlap), _lib.stream_ptr())
        _lib.check(rc, "compressor_pool_fwd")
        ctx.save_for_backward(kv, score, ape, out, lse)
        ctx.cfg = (ratio, head_dim, overlap)
        return out

    @staticmethod
    def backward(ctx, g):
        kv, score, ape, out, lse = ctx.saved_tensors
        ratio, head_dim, overlap = ctx.cfg
        B, S, width = kv.shape
        dkv, dscore = torch.empty_like(kv), torch.empty_like(score)
        g = g.contiguous().float()
        rc = _lib.lib().tb_compressor_pool_bwd(kv.data_ptr(), score.data_ptr(), ape.data_ptr(), out.data_ptr(),
                                               lse.data_ptr(), g.data_ptr(), dkv.data_ptr(), dscore.data_ptr(), B, S,
                                               ratio, head_dim, int(overlap), _lib.stream_ptr())
        _lib.check(rc, "compressor_pool_bwd")
        dape = dscore.view(B * (S // ratio), ratio, width).sum(0) if ctx.needs_input_grad[2] else None
        return dkv, dscore, dape, None, None, None


def compressor_pool(kv: torch.Tensor, score: torch.Tensor, ape: torch.Tensor, ratio: int, head_dim: int,
                    overlap: bool) -> torch.Tensor:
    """kv, score [B, S, width] fp32, ape [ratio, width] fp32 → pooled [B, S / ratio, head_dim] fp32."""
    if _lib.on_device(kv) and kv.dtype == torch.float32 and score.dtype == torch.float32 and head_dim % 4 == 0:
        return _PoolFn.apply(kv, score, ape.float(), ratio, head_dim, overlap)
    return compressor_pool_ref(kv, score, ape.float(), ratio, head_dim, overlap)
