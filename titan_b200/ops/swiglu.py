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
        return _fwd(gate, up, score, rows, H, pitch, limit)

    @staticmethod
    def backward(ctx, gout):
        rows, H, pitch, limit, fused, has_score = ctx.meta
        gout = gout.contiguous()
        saved = ctx.saved_tensors  # read once: activation checkpointing forbids a second unpack
        if fused:
            x = saved[0]
            gate, up = x, x[:, H:]
            dx = torch.empty_like(x)
            dgate, dup = dx, dx[:, H:]
        else:
            gate, up = saved[0], saved[1]
            dgate, dup = torch.empty_like(gate), torch.empty_like(up)
        dscore = torch.empty(rows, dtype=torch.float32, device=gout.device) if has_score else None
        rc = _lib.lib().tb_swiglu_bwd(gout.data_ptr(), gate.data_ptr(), up.data_ptr(), dgate.data_ptr(), dup.data_ptr(),
                                      _lib.ptr(ctx.score32), _lib.ptr(dscore), rows, H, pitch, H, limit,
                                      _lib.dtype_code(gout.dtype), _lib.stream_ptr())
        _lib.check(rc, "swiglu_bwd")
        ds = None
        if has_score:
            orig = saved[-1]
            ds = dscore.to(orig.dtype).view(orig.shape)
        if fused:
            return dx, None, ds, None, None
        return dgate, dup, ds, None, None


def swiglu(gate: torch.Tensor, up: torch.Tensor, score: torch.Tensor | None = None, limit: float = 0.0):
    """silu(gate) * up over the last dim; any leading shape."""
    if not gate.is_cuda:
        return swiglu_ref(gate.reshape(-1, gate.shape[-1]), up.reshape(-1, up.shape[-1]), score, limit).view(gate.shape)
    shape = gate.shape
    out = _SwiGLUFn.apply(gate.reshape(-1, shape[-1]), up.reshape(-1, shape[-1]), score, limit, False)
    return out.view(shape)


def swiglu_fused(x13: torch.Tensor, score: torch.Tensor | None = None, limit: float = 0.0):
    """`x13` [rows, 2H] = gate | up → [rows, H]."""
    if not x13.is_cuda:
        H = x13.shape[-1] // 2
        return swiglu_ref(x13[..., :H], x13[..., H:], score, limit)
    return _SwiGLUFn.apply(x13, None, score, limit, True)
