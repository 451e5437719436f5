"""Row softmax under a selection mask (`csrc/attention/masked_softmax.cu`): ``softmax(scale·S)`` over the allowed
columns, zeros elsewhere, in the storage dtype with fp32 statistics; one read and one write of the logits in forward,
two reads and one write in backward (rows wider than 16384 columns: one more read each).  ``allowed`` has one row per query and is shared by all heads.

Used by the dense form of sparse attention (`ops/dsa.py`), where PyTorch would spend ~10 elementwise passes over the
fp32 [heads, queries, keys] logits.  CPU tensors and odd widths use PyTorch.
"""

from __future__ import annotations

import ctypes

import torch

from titan_b200.ops import _lib

__all__ = ["masked_softmax", "masked_softmax_ref"]

_DECLARED = False
_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def masked_softmax_ref(s: torch.Tensor, allowed: torch.Tensor, scale: float = 1.0,
                       sink: torch.Tensor | None = None) -> torch.Tensor:
    """s [H, Sc, T], allowed [Sc, T] bool, sink [H] | None → probabilities [H, Sc, T] in s.dtype (rows without allowed
    key: zeros).  ``sink`` is one extra logit per head that only joins the denominator."""
    x = (s.float() * scale).masked_fill(~allowed.unsqueeze(0), float("-inf"))
    if sink is not None:
        x = torch.cat([x, sink.float().view(-1, 1, 1).expand(-1, x.shape[1], 1)], dim=-1)
        return torch.softmax(x, dim=-1)[..., :-1].to(s.dtype)
    return torch.nan_to_num(torch.softmax(x, dim=-1)).to(s.dtype)


def _declare():
    global _DECLARED
    if not _DECLARED:
        P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        _lib.declare("tb_masked_softmax_fwd", [P, P, P, LL, I, I, F, P, I, P])
        _lib.declare("tb_masked_softmax_bwd", [P, P, P, LL, I, F, P, I, P])
        _DECLARED = True


class _MaskedSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, s, allowed, scale, sink):
        _declare()
        H, Sc, T = s.shape
        s = s.contiguous()
        mask = allowed.contiguous().view(torch.uint8)
        p = torch.empty_like(s)
        sk = sink.detach().float().contiguous() if sink is not None else None
        rc = _lib.lib().tb_masked_softmax_fwd(s.data_ptr(), mask.data_ptr(), p.data_ptr(), H * Sc, T, Sc, float(scale),
                                              _lib.ptr(sk), _lib.dtype_code(s.dtype), _lib.stream_ptr())
        _lib.check(rc, "masked_softmax_fwd")
        ctx.save_for_backward(p)
        ctx.scale, ctx.has_sink = float(scale), sink is not None
        ctx.sink_dtype = sink.dtype if sink is not None else None
        return p

    @staticmethod
    def backward(ctx, g):
        (p,) = ctx.saved_tensors
        H, Sc, T = p.shape
        g = g.contiguous().to(p.dtype)
        ds = torch.empty_like(p)
        rows = torch.empty(H * Sc, dtype=torch.float32, device=p.device) if ctx.has_sink else None
        rc = _lib.lib().tb_masked_softmax_bwd(p.data_ptr(), g.data_ptr(), ds.data_ptr(), H * Sc, T, ctx.scale,
                                              _lib.ptr(rows), _lib.dtype_code(p.dtype), _lib.stream_ptr())
        _lib.check(rc, "masked_softmax_bwd")
        dsink = rows.view(H, Sc).sum(1).to(ctx.sink_dtype) if ctx.has_sink else None
        return ds, None, None, dsink


def masked_softmax(s: torch.Tensor, allowed: torch.Tensor, scale: float = 1.0,
                   sink: torch.Tensor | None = None) -> torch.Tensor:
    """s [H, Sc, T] logits, allowed [Sc, T] bool, sink [H] | None → probabilities [H, Sc, T] in s.dtype."""
    T = s.shape[-1]
    vec = 4 if s.dtype == torch.float32 else 8
    if _lib.on_device(s) and s.dim() == 3 and s.dtype in _DTYPES and T % vec == 0 \
            and allowed.dtype == torch.bool and allowed.shape == s.shape[1:]:
        return _MaskedSoftmax.apply(s, allowed, scale, sink)
    return masked_softmax_ref(s, allowed, scale, sink)
