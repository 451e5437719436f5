"""Causal flash attention (dense, GQA) on the tcgen05 forward kernel.

Forward: `tb_flash_attn_fwd` (csrc/attention/flash_fwd.cu) for bf16, head_dim 128, sequence a multiple of 128,
tensors in ``[B, S, H, D]`` memory order (the order the projections produce: no transposes or copies).  Everything
else, and the backward, goes to the library attention: the backward recomputes the library forward for its saved
statistics and differentiates that (same math; the gradient kernels of this op are not written yet).

Parity: the reference's fused attention op (K7 `npu_fusion_attention`, causal, BSND) behind its attention wrapper.
"""

from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from titan_b200.ops import _lib

__all__ = ["flash_attention", "flash_attention_supported"]

_DECLARED = False


def _declare():
    global _DECLARED
    if not _DECLARED:
        P, I, Fl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        _lib.declare("tb_flash_attn_fwd", [P, P, P, P, P, I, I, I, I, I, Fl, P, P])
        _DECLARED = True


def flash_attention_supported(q: torch.Tensor, k: torch.Tensor) -> bool:
    """q [B, H, S, D] / k [B, Hkv, S, D] views of [B, S, H, D] storage."""
    return ((q.is_cuda or q.is_meta) and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and q.shape[2] % 128 == 0
            and q.shape[2] == k.shape[2] and q.shape[1] % k.shape[1] == 0)


def _bshd(t: torch.Tensor) -> torch.Tensor:
    """[B, H, S, D] (any strides) → contiguous [B, S, H, D] (no copy when it already is a transposed view of that)."""
    return t.transpose(1, 2).contiguous()


def _library(q, k, v, scale):
    return F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=q.shape[1] != k.shape[1])


def _flash_fwd_launch(q, k, v, scale):
    """q [B, H, S, D], k / v [B, Hkv, S, D] → (out [B, H, S, D] as a view of [B, S, H, D] storage, lse [B, H, S])."""
    _declare()
    qb, kb, vb = _bshd(q), _bshd(k), _bshd(v)
    B, S, H, D = qb.shape
    out = torch.empty_like(qb)
    lse = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    rc = _lib.lib().tb_flash_attn_fwd(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                      B, S, H, kb.shape[2], D, float(scale), _lib.shared_status().ptr,
                                      _lib.stream_ptr())
    _lib.check(rc, "flash_attn_fwd")
    return out.transpose(1, 2), lse


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        from titan_b200.ops.registry import ops

        out, lse = ops.flash_attention_fwd(q, k, v, float(scale))
        ctx.save_for_backward(q, k, v)
        ctx.scale = scale
        ctx.lse = lse
        return out

    @staticmethod
    def backward(ctx, g):
        q, k, v = ctx.saved_tensors
        with torch.enable_grad():
            qd, kd, vd = (t.detach().requires_grad_() for t in (q, k, v))
            o = _library(qd, kd, vd, ctx.scale)
        dq, dk, dv = torch.autograd.grad(o, (qd, kd, vd), g)
        return dq, dk, dv, None


def flash_attention(q, k, v, *, scale: float | None = None):
    """q [B, H, S, D], k / v [B, Hkv, S, D] → [B, H, S, D]; causal."""
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    if not flash_attention_supported(q, k):
        return _library(q, k, v, scale)
    return _FlashFn.apply(q, k, v, scale)
