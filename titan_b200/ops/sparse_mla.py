"""Sparse multi-head latent attention on the tcgen05 kernel (`csrc/attention/sparse_mla_fwd.cu`).

``sparse_mla_forward(q, kv, idx, scale, dv)`` attends every query to its selected rows of the shared one-head KV latent
only: the kernel gathers 128 selected rows at a time into shared memory and runs both contractions on the tensor
cores, so memory and work are O(S * top-k) however long the key stream is.  It returns the output, the log-sum-exp and
the head-summed probabilities (the teacher of the lightning indexer's KL loss), all exact (two passes over the keys).

`SparseMLAFunction` adds autograd: the backward kernel (`csrc/attention/sparse_mla_bwd.cu`) recomputes the
probabilities from the saved log-sum-exp on the same gathered tiles, keeps dQ in tensor memory and adds the latent's
gradient row by row with bulk reductions, so nothing of size [S, T] exists in either direction.  A chunked PyTorch
backward (`sparse_mla_backward_ref`) is the oracle of its test.

Parity: `npu_sparse_flash_attention` with `softmax_lse` output (torchtitan_npu/converters/kernels/dsa.py:195-277) and
`sparse_flash_mla` / `sparse_flash_mla_grad` (converters/kernels/npu_smla.py:59-1348).
"""

from __future__ import annotations

import ctypes

import torch

from titan_b200.ops import _lib

__all__ = ["sparse_mla_supported", "sparse_mla_forward", "sparse_mla_forward_ref", "sparse_mla_backward",
           "sparse_mla_backward_ref", "sparse_mla"]

_DECLARED = False


def _declare():
    global _DECLARED
    if not _DECLARED:
        P, I, Fl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        _lib.declare("tb_sparse_mla_fwd", [P, P, P, P, P, P, P, I, I, I, I, I, I, Fl, P, P])
        _lib.declare("tb_sparse_mla_bwd", [P, P, P, P, P, P, P, P, I, I, I, I, I, I, Fl, P, P])
        _lib.declare("tb_sparse_mla_fwd_set_pipelined", [I])
        _DECLARED = True


def set_pipelined(on: bool) -> None:
    """Forward kernel selection: False (default) is the single-tile kernel; True uses the half-tile ring where it
    applies (logits fit in tensor memory, value width a multiple of 256).  The ring overlaps the copies with the
    products but doubles the product / wait round trips and measures slightly slower; it is kept and tested."""
    _declare()
    _lib.check(_lib.lib().tb_sparse_mla_fwd_set_pipelined(int(bool(on))), "sparse_mla_fwd_set_pipelined")


def sparse_mla_supported(q: torch.Tensor, kv: torch.Tensor, idx: torch.Tensor, dv: int) -> bool:
    """q [S, H, Dq], kv [T, Dq], idx [S, K]."""
    H, dq = q.shape[1], q.shape[2]
    return ((q.is_cuda or q.is_meta) and q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and H % 16 == 0
            and dq % 64 == 0 and dq <= 576 and dv % 128 == 0 and dv <= min(512, dq) and idx.shape[1] % 128 == 0)


def sparse_mla_forward_ref(q, kv, idx, scale: float, dv: int, sink: torch.Tensor | None = None):
    """fp32 oracle: gather, softmax over the selected keys (+ an optional per-head sink logit in the denominator)."""
    S, H, _ = q.shape
    safe = idx.clamp_min(0).long()
    ksel = kv.float()[safe]                                  # [S, K, Dq]
    s = torch.einsum("shd,skd->shk", q.float(), ksel) * scale
    s = s.masked_fill((idx < 0).unsqueeze(1), float("-inf"))
    if sink is not None:
        s_all = torch.cat([s, sink.float().view(1, H, 1).expand(S, H, 1)], dim=-1)
        lse = torch.logsumexp(s_all, dim=-1)
    else:
        lse = torch.logsumexp(s, dim=-1)
    p = torch.nan_to_num(torch.exp(s - lse.unsqueeze(-1)))
    out = torch.einsum("shk,skd->shd", p, ksel[..., :dv])
    return out.to(q.dtype), lse, p.sum(1)


def sparse_mla_forward(q, kv, idx, scale: float, dv: int, sink: torch.Tensor | None = None, want_teacher=True):
    """q [S, H, Dq] bf16, kv [T, Dq] bf16 (values = first ``dv`` columns), idx [S, K] int32 (-1 = empty slot)
    → (out [S, H, dv], lse [S, H] fp32, teacher [S, K] fp32 or None)."""
    _declare()
    S, H, dq = q.shape
    T, K = kv.shape[0], idx.shape[1]
    q, kv = q.contiguous(), kv.contiguous()
    idx = idx.to(torch.int32).contiguous()
    out = torch.empty(S, H, dv, dtype=q.dtype, device=q.device)
    lse = torch.empty(S, H, dtype=torch.float32, device=q.device)
    teacher = torch.zeros(S, K, dtype=torch.float32, device=q.device) if want_teacher else None
    sk = sink.float().contiguous() if sink is not None else None
    rc = _lib.lib().tb_sparse_mla_fwd(q.data_ptr(), kv.data_ptr(), idx.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                      _lib.ptr(teacher), _lib.ptr(sk), S, H, T, K, dq, dv, float(scale),
                                      _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "sparse_mla_fwd")
    return out, lse, teacher


class SparseMLAFunction(torch.autograd.Function):
    """(q, kv, idx) → (out, teacher, lse).  ``kv`` carries keys AND values (first ``dv`` columns); its gradient sums
    both roles.  `teacher` and `lse` carry no gradient."""

    @staticmethod
    def forward(ctx, q, kv, idx, scale, dv, sink, chunk):
        from titan_b200.ops.registry import ops

        out, lse, teacher = ops.sparse_mla_fwd(q, kv, idx.to(torch.int32), float(scale), dv, sink)
        ctx.save_for_backward(q, kv, idx, lse, out, sink if sink is not None else torch.empty(0, device=q.device))
        ctx.scale, ctx.dv, ctx.chunk, ctx.has_sink = scale, dv, chunk, sink is not None
        ctx.mark_non_differentiable(teacher, lse)
        return out, teacher, lse

    @staticmethod
    def backward(ctx, g_out, _gt, _gl):
        q, kv, idx, lse, out, sink = ctx.saved_tensors
        H = q.shape[1]
        delta = (g_out.float() * out.float()).sum(-1)                    # [S, H]
        if KERNEL_BACKWARD:
            dq_, dkv = sparse_mla_backward(q, kv, idx, g_out, lse, delta, ctx.scale, ctx.dv)
        else:
            dq_, dkv = sparse_mla_backward_ref(q, kv, idx, g_out, lse, delta, ctx.scale, ctx.dv, ctx.chunk)
        dsink = None
        if ctx.has_sink:   # probability mass on the sink times -delta, summed over the queries
            dsink = -(torch.exp(sink.float().view(1, H) - lse) * delta).sum(0).to(sink.dtype)
        return dq_, dkv.to(kv.dtype), None, None, None, dsink, None


KERNEL_BACKWARD = True  # False: the chunked PyTorch backward below (the oracle of the kernel's test)


def sparse_mla_backward(q, kv, idx, g_out, lse, delta, scale: float, dv: int):
    """Gradients of queries and latent on the tensor cores (`csrc/attention/sparse_mla_bwd.cu`):
    → (dq [S, H, Dq] bf16, dkv [T, Dq] fp32)."""
    if not q.is_meta:
        _declare()
    S, H, dq = q.shape
    T, K = kv.shape[0], idx.shape[1]
    q, kv, g_out = q.contiguous(), kv.contiguous(), g_out.contiguous()
    idx = idx.to(torch.int32).contiguous()
    dq_ = torch.empty_like(q)
    dkv = torch.zeros(T, dq, dtype=torch.float32, device=kv.device)
    if q.is_meta:   # shapes only (memory simulation)
        _lib.note_skipped_launch("tb_sparse_mla_bwd", (None,) * 8 + (S, H, T, K, dq, dv))
        return dq_, dkv
    rc = _lib.lib().tb_sparse_mla_bwd(q.data_ptr(), kv.data_ptr(), idx.data_ptr(), g_out.data_ptr(),
                                      lse.contiguous().data_ptr(), delta.contiguous().data_ptr(), dq_.data_ptr(),
                                      dkv.data_ptr(), S, H, T, K, dq, dv, float(scale),
                                      _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "sparse_mla_bwd")
    return dq_, dkv


def sparse_mla_backward_ref(q, kv, idx, g_out, lse, delta, scale: float, dv: int, chunk: int = 128):
    """The same gradients in PyTorch, ``chunk`` queries at a time (memory O(chunk * K * Dq))."""
    S, H, dq = q.shape
    dq_ = torch.empty_like(q)
    dkv = torch.zeros(kv.shape[0], dq, dtype=torch.float32, device=kv.device)
    for s0 in range(0, S, chunk):
        s1 = min(s0 + chunk, S)
        ix = idx[s0:s1]
        safe = ix.clamp_min(0).long()
        ksel = kv[safe]                                              # [sc, K, Dq] storage dtype
        sc = torch.einsum("shd,skd->shk", q[s0:s1], ksel).float() * scale
        p = torch.exp(sc - lse[s0:s1].unsqueeze(-1)).masked_fill((ix < 0).unsqueeze(1), 0.0)
        go = g_out[s0:s1]
        dp = torch.einsum("shd,skd->shk", go, ksel[..., :dv]).float()
        ds = (p * (dp - delta[s0:s1].unsqueeze(-1)) * scale).to(q.dtype)
        dq_[s0:s1] = torch.einsum("shk,skd->shd", ds, ksel)
        dk_rows = torch.einsum("shk,shd->skd", ds, q[s0:s1]).float()  # score path, [sc, K, Dq]
        dk_rows[..., :dv] += torch.einsum("shk,shd->skd", p.to(q.dtype), go).float()   # value path
        dkv.index_add_(0, safe.reshape(-1), dk_rows.reshape(-1, dq))
    return dq_, dkv


def sparse_mla(q, kv, idx, scale: float, dv: int, sink: torch.Tensor | None = None, chunk: int = 128):
    """Differentiable sparse MLA → (out [S, H, dv], teacher [S, K], lse [S, H])."""
    return SparseMLAFunction.apply(q, kv, idx, scale, dv, sink, chunk)
