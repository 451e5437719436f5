"""Causal flash attention (dense, GQA, optionally per document of a packed sequence) on tcgen05 kernels.

Forward `tb_flash_attn_fwd` (csrc/attention/flash_fwd.cu) and backward `tb_flash_attn_bwd`
(csrc/attention/flash_bwd.cu) for bf16, head_dim 128, sequence a multiple of 128, tensors in ``[B, S, H, D]`` memory
order (the order the projections produce: no transposes or copies).  Packed sequences pass ``seq_start`` ([B, S]
int32: the position of the first token of each token's document); a query then sees the keys of its own document
only, inside the same kernels.  Other shapes go to the library attention.

Parity: the reference's fused attention op and its gradient (K7 `npu_fusion_attention`, causal, BSND; the packed TND
form of torchtitan_npu/models/common/npu_varlen_attention.py:42-97) behind its attention wrappers.
"""

from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from titan_b200.ops import _lib

__all__ = ["flash_attention", "flash_attention_supported", "seq_start_from_cu_seqlens"]

_DECLARED = False


def _declare():
    global _DECLARED
    if not _DECLARED:
        P, I, Fl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        _lib.declare("tb_flash_attn_fwd", [P, P, P, P, P, P, I, I, I, I, I, Fl, P, P])
        _lib.declare("tb_flash_attn_bwd", [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, Fl, P, P])
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


def seq_start_from_cu_seqlens(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    """Cumulative document ends ``[0, e1, e2, ...]`` of one packed stream of ``total`` tokens → [total] int32 with the
    start position of each token's document (tokens past the last boundary form one more document)."""
    cu = cu_seqlens.to(torch.int64)
    pos = torch.arange(total, device=cu.device)
    doc = torch.searchsorted(cu, pos, right=True) - 1
    return cu[doc.clamp(min=0)].to(torch.int32)


def _check_seq_start(seq_start, B, S):
    if seq_start is None:
        return None
    if seq_start.numel() != B * S:
        raise ValueError(f"seq_start must have one entry per token ({B} x {S}), got {tuple(seq_start.shape)}")
    return seq_start.to(torch.int32).contiguous()


def _flash_fwd_launch(q, k, v, scale, seq_start=None):
    """q [B, H, S, D], k / v [B, Hkv, S, D] → (out [B, H, S, D] as a view of [B, S, H, D] storage, lse [B, H, S])."""
    _declare()
    qb, kb, vb = _bshd(q), _bshd(k), _bshd(v)
    B, S, H, D = qb.shape
    out = torch.empty_like(qb)
    lse = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    ss = _check_seq_start(seq_start, B, S)
    rc = _lib.lib().tb_flash_attn_fwd(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                      _lib.ptr(ss), B, S, H, kb.shape[2], D, float(scale),
                                      _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "flash_attn_fwd")
    return out.transpose(1, 2), lse


def _flash_bwd_launch(q, k, v, out, lse, g, scale, seq_start=None):
    """→ (dq, dk, dv) as [B, H, S, D] views of [B, S, H, D] storage."""
    _declare()
    qb, kb, vb, ob, gb = _bshd(q), _bshd(k), _bshd(v), _bshd(out), _bshd(g)
    B, S, H, D = qb.shape
    delta = torch.einsum("bshd,bshd->bhs", gb.float(), ob.float()).contiguous()   # rowsum(dO * O), [B, H, S]
    dq32 = torch.zeros(B, S, H, D, dtype=torch.float32, device=q.device)
    dk, dv = torch.empty_like(kb), torch.empty_like(vb)
    ss = _check_seq_start(seq_start, B, S)
    rc = _lib.lib().tb_flash_attn_bwd(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), gb.data_ptr(),
                                      lse.contiguous().data_ptr(), delta.data_ptr(), _lib.ptr(ss), dk.data_ptr(),
                                      dv.data_ptr(), dq32.data_ptr(), B, S, H, kb.shape[2], D, float(scale),
                                      _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "flash_attn_bwd")
    return dq32.to(q.dtype).transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)


KERNEL_BACKWARD = True  # False: differentiate the library attention instead (dense causal only)


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, seq_start):
        from titan_b200.ops.registry import ops

        out, lse = ops.flash_attention_fwd(q, k, v, float(scale), seq_start)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale, ctx.seq_start = scale, seq_start
        return out

    @staticmethod
    def backward(ctx, g):
        from titan_b200.ops.registry import ops

        q, k, v, out, lse = ctx.saved_tensors
        if KERNEL_BACKWARD or ctx.seq_start is not None:
            dq, dk, dv = ops.flash_attention_bwd(q, k, v, out, lse, g, float(ctx.scale), ctx.seq_start)
            return dq, dk, dv, None, None
        with torch.enable_grad():
            qd, kd, vd = (t.detach().requires_grad_() for t in (q, k, v))
            o = _library(qd, kd, vd, ctx.scale)
        dq, dk, dv = torch.autograd.grad(o, (qd, kd, vd), g)
        return dq, dk, dv, None, None


def flash_attention(q, k, v, *, scale: float | None = None, seq_start: torch.Tensor | None = None):
    """q [B, H, S, D], k / v [B, Hkv, S, D] → [B, H, S, D]; causal, and per document when ``seq_start`` ([B, S] int32,
    first position of each token's document) is given."""
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    if not flash_attention_supported(q, k):
        if seq_start is not None:
            raise ValueError("packed-document attention needs bf16, head_dim 128 and a sequence multiple of 128")
        return _library(q, k, v, scale)
    return _FlashFn.apply(q, k, v, scale, seq_start)
