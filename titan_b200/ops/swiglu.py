"""SwiGLU (+clamp, +per-row score): sm_100a kernel with autograd + oracle.

``swiglu(gate, up)`` for separate projections; ``swiglu_fused(x13, score, limit)`` for a fused
``[rows, 2H]`` buffer (``gate | up``) as produced by a grouped GEMM on ``w13``.

Parity: reference expert activation (torchtitan_npu/converters/kernels/gmm.py:87-104,
models/deepseek_v4/moe.py:216-220).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from titan_b200.ops import _lib

__all__ = ["swiglu", "swiglu_fused", "swiglu_ref"]


def swiglu_ref(gate, up, score=None, limit: float = 0.0):
    g, u = gate.float(), up.float()
    if limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    out = F.silu(g) * u
    if score is not None:
        out = out * score.float().reshape(-1, 1)
    return out.to(gate.dtype)


def _fwd(gate, up, score, rows, H, in_pitch, limit):
    out = torch.empty(rows, H, dtype=gate.dtype, device=gate.device)
    rc = _lib.lib().tb_swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(), _lib.ptr(score), rows, H, in_pitch, H,
                                  float(limit), _lib.dtype_code(gate.dtype), _lib.stream_ptr())
    _lib.check(rc, "swiglu_fwd")
    return out


def _bwd(gout, gate, up, score, rows, H, pitch, limit):
    """→ (dgate, dup, dscore).  ``up is None``: gate and up are the halves of one [rows, 2H] tensor and the gradient
    comes back as one tensor of that shape in ``dgate`` (``dup`` is empty).  Without a score ``dscore`` is empty."""
    if up is None:
        dgate = torch.empty_like(gate)
        up_, dup_, dup = gate[:, H:], dgate[:, H:], gate.new_empty(0)
    else:
        dgate, dup = torch.empty_like(gate), torch.empty_like(up)
        up_, dup_ = up, dup
    dscore = torch.empty(rows, dtype=torch.float32, device=gout.device) if score is not None else gout.new_empty(0)
    rc = _lib.lib().tb_swiglu_bwd(gout.data_ptr(), gate.data_ptr(), up_.data_ptr(), dgate.data_ptr(), dup_.data_ptr(),
                                  _lib.ptr(score), dscore.data_ptr() if score is not None else None, rows, H, pitch, H,
                                  float(limit), _lib.dtype_code(gout.dtype), _lib.stream_ptr())
    _lib.check(rc, "swiglu_bwd")
    return dgate, dup, dscore


class _SwiGLUFn(torch.autograd.Function):
    """`fused` = gate and up are the two halves of one [rows, 2H] tensor."""

    @staticmethod
    def forward(ctx, a, b, score, limit, fused):
        if fused:
            x = a.contiguous()
            rows, H = x.shape[0], x.shape[1] // 2
            gate, up, pitch = x, x[:, H:], 2 * H
            ctx.save_for_backward(x, score if score is not None else torch.empty(0))
        else:
            gate, up = a.contiguous(), b.contiguous()
            rows, H = gate.shape[0], gate.shape[1]
            pitch = H
            ctx.save_for_backward(gate, up, score if score is not None else torch.empty(0))
        if score is not None:
            score = score.reshape(-1).float().contiguous()
        ctx.meta = (rows, H, pitch, float(limit), fused, score is not None)
        ctx.score32 = score
        from titan_b200.ops.registry import ops

        return ops.swiglu_fwd(gate, None if fused else up, score, rows, H, pitch, float(limit))

    @staticmethod
    def backward(ctx, gout):
        rows, H, pitch, limit, fused, has_score = ctx.meta
        gout = gout.contiguous()
        saved = ctx.saved_tensors  # read once: activation checkpointing forbids a second unpack
        from titan_b200.ops.registry import ops

        if fused:
            dx, _, dscore = ops.swiglu_bwd(gout, saved[0], None, ctx.score32, rows, H, pitch, limit)
        else:
            dgate, dup, dscore = ops.swiglu_bwd(gout, saved[0], saved[1], ctx.score32, rows, H, pitch, limit)
        ds = None
        if has_score:
            orig = saved[-1]
            ds = dscore.to(orig.dtype).view(orig.shape)
        if fused:
            return dx, None, ds, None, None
        return dgate, dup, ds, None, None


def swiglu(gate: torch.Tensor, up: torch.Tensor, score: torch.Tensor | None = None, limit: float = 0.0):
    """silu(gate) * up over the last dim; any leading shape."""
    if not (gate.is_cuda or gate.is_meta):
        return swiglu_ref(gate.reshape(-1, gate.shape[-1]), up.reshape(-1, up.shape[-1]), score, limit).view(gate.shape)
    shape = gate.shape
    out = _SwiGLUFn.apply(gate.reshape(-1, shape[-1]), up.reshape(-1, shape[-1]), score, limit, False)
    return out.view(shape)


def swiglu_fused(x13: torch.Tensor, score: torch.Tensor | None = None, limit: float = 0.0):
    """`x13` [rows, 2H] = gate | up → [rows, H]."""
    if not (x13.is_cuda or x13.is_meta):
        H = x13.shape[-1] // 2
        return swiglu_ref(x13[..., :H], x13[..., H:], score, limit)
    return _SwiGLUFn.apply(x13, None, score, limit, True)
