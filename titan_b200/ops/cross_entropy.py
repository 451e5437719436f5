"""Fused softmax cross-entropy over large vocabularies (sm_100a kernel) + oracle.

``cross_entropy_sum(logits, labels)`` returns the *sum* of token losses (the trainer divides by the
global token count).  Logits stay in their storage dtype; statistics are fp32 inside the kernel.
Backward writes ``(softmax - onehot) * upstream`` over the logits buffer when it is safe to do so
(the logits are an intermediate nobody else reads), saving a [T, V] allocation.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from titan_b200.ops import _lib

__all__ = ["cross_entropy_sum", "cross_entropy_ref"]

IGNORE_INDEX = -100


def cross_entropy_ref(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = IGNORE_INDEX) -> torch.Tensor:
    return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1), reduction="sum",
                           ignore_index=ignore_index)


def _fwd_rows(x, labels, ignore_index):
    """x [rows, V] (unit inner stride), labels [rows] int64 → (per-row loss, per-row log-sum-exp), both fp32."""
    rows, V, pitch = x.shape[0], x.shape[1], x.stride(0)
    loss = torch.empty(rows, dtype=torch.float32, device=x.device)
    lse = torch.empty(rows, dtype=torch.float32, device=x.device)
    status = _lib.shared_status()
    rc = _lib.lib().tb_cross_entropy_fwd(x.data_ptr(), labels.data_ptr(), loss.data_ptr(), lse.data_ptr(), rows, V,
                                         pitch, ignore_index, _lib.dtype_code(x.dtype), status.ptr, _lib.stream_ptr())
    _lib.check(rc, "cross_entropy_fwd")
    return loss, lse


def _bwd_rows(x, labels, lse, gscale, ignore_index, inplace):
    """Gradient of the summed loss w.r.t. the logits, scaled by ``gscale``; written over ``x`` when ``inplace``."""
    rows, V, pitch = x.shape[0], x.shape[1], x.stride(0)
    d = x if inplace else torch.empty_like(x)
    rc = _lib.lib().tb_cross_entropy_bwd(x.data_ptr(), labels.data_ptr(), lse.data_ptr(), gscale.data_ptr(),
                                         d.data_ptr(), rows, V, d.stride(0), ignore_index, _lib.dtype_code(x.dtype),
                                         _lib.stream_ptr())
    _lib.check(rc, "cross_entropy_bwd")
    return d


class _CEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index, inplace_backward):
        V = logits.shape[-1]
        x = logits.reshape(-1, V)
        if not x.is_contiguous():
            x = x.contiguous()
        rows, pitch = x.shape[0], x.stride(0)
        labels = labels.reshape(-1).to(torch.int64).contiguous()
        from titan_b200.ops.registry import ops

        loss, lse = ops.cross_entropy_fwd(x, labels, ignore_index)
        ctx.save_for_backward(x, labels, lse)
        ctx.meta = (rows, V, pitch, ignore_index, inplace_backward, logits.shape)
        return loss.sum()

    @staticmethod
    def backward(ctx, g):
        x, labels, lse = ctx.saved_tensors
        rows, V, pitch, ignore_index, inplace, shape = ctx.meta
        gscale = g.reshape(1).float().contiguous()
        from titan_b200.ops.registry import ops

        if inplace:
            ops.cross_entropy_bwd_(x, labels, lse, gscale, ignore_index)
            d = x
        else:
            d = ops.cross_entropy_bwd(x, labels, lse, gscale, ignore_index)
        return d.view(shape), None, None, None


def cross_entropy_sum(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = IGNORE_INDEX,
                      inplace_backward: bool = False) -> torch.Tensor:
    if not (logits.is_cuda or logits.is_meta):
        return cross_entropy_ref(logits, labels, ignore_index)
    return _CEFn.apply(logits, labels, ignore_index, inplace_backward)
