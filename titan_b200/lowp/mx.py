"""MX (microscaling) quantisation: blocks of 32 values share one power-of-two scale (e8m0), elements are e4m3.

* `mx_quantize(x, axis, round_mode)` → ``(q, scales)``: ``q`` has x's shape (float8_e4m3fn), ``scales`` is uint8 with
  the quantised axis divided by 32.  ``axis=-1`` blocks run along rows (the contraction dim of ``[M, K]``); ``axis=-2``
  blocks run down 32 consecutive rows (operands contracted over their first dim).
* `mx_quantize_dual(x)` → ``(q1, s1, q2t, s2t)`` from ONE read of ``x [R, C]``: the row-blocked pair of ``axis=-1`` and
  the column-blocked pair written TRANSPOSED (``q2t [C, R]``, ``s2t [C, R/32]``), i.e. the K-major operand of a GEMM
  that contracts over R.  Forward and backward of an MX linear need both views of every operand.
* `mx_dequantize(q, scales, axis)` → bf16 (exact: e4m3 × 2^e fits bf16).
* round modes: ``"rceil"`` picks the smallest power of two that keeps the block maximum ≤ 448 (no clipping);
  ``"floor"`` is the OCP rule ``floor(log2 amax) − 8`` (the top of a block may saturate).

CUDA bf16 / fp16 inputs run the sm_100a kernels (`csrc/lowp/mx_quant.cu`); everything else takes the PyTorch statement
below, which is also the oracle of the kernel tests.

Parity: `npu_dynamic_mx_quant(axis, dst_type=float8_e4m3fn, scale_alg)` (torchtitan_npu/patches/torchao_npu/
mx_linear.py:38-99; experiments/ao_npu/torchao_npu/ops/mx_ops.py, quantization/quant_configs.py:24-61).
"""

from __future__ import annotations

import ctypes

import torch

from titan_b200.ops import _lib

__all__ = ["mx_quantize", "mx_dequantize", "mx_quantize_ref", "mx_dequantize_ref", "mx_fake_quantize", "BLOCK", "sqnr",
           "mx_quantize_dual"]

BLOCK = 32
E4M3_MAX = 448.0
_DECLARED = False


def _declare():
    global _DECLARED
    if not _DECLARED:
        P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        _lib.declare("tb_mx_quantize", [P, P, P, LL, I, I, I, I, P])
        _lib.declare("tb_mx_dequantize", [P, P, P, LL, I, I, P])
        _lib.declare("tb_mx_quantize_dual", [P, P, P, P, P, LL, I, I, I, I, P])
        _DECLARED = True


def _exponent(amax: torch.Tensor, round_mode: str) -> torch.Tensor:
    safe = amax.clamp_min(torch.finfo(torch.float32).tiny)
    if round_mode == "rceil":
        e = torch.ceil(torch.log2(safe / E4M3_MAX))
        # log2 of exact powers of two can land a hair above the integer: re-check the bound
        e = torch.where(safe * torch.exp2(-(e - 1)) <= E4M3_MAX, e - 1, e)
    elif round_mode == "floor":
        e = torch.floor(torch.log2(safe)) - 8
    else:
        raise ValueError(f"unknown MX round mode {round_mode!r} (rceil | floor)")
    e = e.clamp(-127, 127)
    return torch.where(amax > 0, e, torch.full_like(e, -127))


def mx_quantize_ref(x: torch.Tensor, axis: int = -1, round_mode: str = "rceil"):
    if axis not in (-1, -2):
        raise ValueError("axis must be -1 or -2")
    xt = x.float() if axis == -1 else x.float().transpose(-1, -2)
    if xt.shape[-1] % BLOCK:
        raise ValueError(f"the quantised axis ({xt.shape[-1]}) must be a multiple of {BLOCK}")
    blocks = xt.reshape(*xt.shape[:-1], -1, BLOCK)
    e = _exponent(blocks.abs().amax(-1), round_mode)
    q = (blocks * torch.exp2(-e).unsqueeze(-1)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    q = q.reshape(xt.shape)
    s = (e + 127).to(torch.uint8)
    if axis == -2:
        q, s = q.transpose(-1, -2).contiguous(), s.transpose(-1, -2).contiguous()
    return q, s


def mx_dequantize_ref(q: torch.Tensor, scales: torch.Tensor, axis: int = -1, dtype=torch.bfloat16):
    s = torch.exp2(scales.float() - 127.0)
    s = s.repeat_interleave(BLOCK, dim=-1 if axis == -1 else -2)
    return (q.float() * s).to(dtype)


def _kernel_ok(x: torch.Tensor, axis: int) -> bool:
    return ((x.is_cuda or x.is_meta) and x.dtype in (torch.bfloat16, torch.float16) and x.dim() == 2 and x.is_contiguous()
            and x.shape[1] % 8 == 0 and x.shape[-1 if axis == -1 else -2] % BLOCK == 0
            and (axis == -1 or x.shape[0] // BLOCK <= 65535))


def mx_quantize(x: torch.Tensor, axis: int = -1, round_mode: str = "rceil"):
    """x [..., R, C] → (q float8_e4m3fn [..., R, C], scales uint8 [..., R, C/32] or [..., R/32, C])."""
    if x.dim() > 2 and axis == -1:
        q, s = mx_quantize(x.reshape(-1, x.shape[-1]), axis, round_mode)
        return q.view(x.shape), s.view(*x.shape[:-1], -1)
    if not _kernel_ok(x, axis):
        return mx_quantize_ref(x, axis, round_mode)
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    s = torch.empty((rows, cols // BLOCK) if axis == -1 else (rows // BLOCK, cols), dtype=torch.uint8, device=x.device)
    if x.is_meta:   # shapes only (memory simulation)
        _lib.note_skipped_launch("tb_mx_quantize", (None, None, None, rows, cols))
        return q.view(torch.float8_e4m3fn), s
    _declare()
    rc = _lib.lib().tb_mx_quantize(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows, cols, axis,
                                   {"floor": 0, "rceil": 1}[round_mode], _lib.dtype_code(x.dtype), _lib.stream_ptr())
    _lib.check(rc, "mx_quantize")
    return q.view(torch.float8_e4m3fn), s


def mx_quantize_dual(x: torch.Tensor, round_mode: str = "rceil", *, rows: bool = True, transposed: bool = True,
                     atoms: bool = False):
    """x [R, C] (R, C multiples of 32) → ``(q1 [R, C], s1 [R, C/32], q2t [C, R], s2t [C, R/32])``; a view that is not
    asked for (``rows=False`` / ``transposed=False``) comes back as ``None, None``.  ``q2t, s2t`` equal
    ``mx_quantize(x.t().contiguous(), -1)``.  ``atoms=True`` (both dims multiples of 128) returns the scales in the
    packed 512-byte atom order of the block-scaled GEMM (`ops.mxfp8_gemm.pack_scale_atoms`): ``s1 [R/128, C/128, 512]``,
    ``s2t [C/128, R/128, 512]``, ready for ``mxfp8_gemm(..., packed=True)`` with no repacking pass.

    Parity: `npu_dynamic_mx_quant_with_dual_axis` as used by experiments/ao_npu/torchao_npu/ops/mx_ops.py:62-194."""
    if x.dim() != 2 or x.shape[0] % BLOCK or x.shape[1] % BLOCK:
        raise ValueError(f"mx_quantize_dual wants a 2-D tensor with both dims multiples of {BLOCK}, got {tuple(x.shape)}")
    if not (rows or transposed):
        raise ValueError("mx_quantize_dual: ask for at least one view")
    if atoms and (x.shape[0] % 128 or x.shape[1] % 128):
        raise ValueError("mx_quantize_dual(atoms=True) needs both dims to be multiples of 128")
    if not ((x.is_cuda or x.is_meta) and x.dtype in (torch.bfloat16, torch.float16)):
        q1, s1 = mx_quantize_ref(x, -1, round_mode) if rows else (None, None)
        q2t, s2t = mx_quantize_ref(x.t().contiguous(), -1, round_mode) if transposed else (None, None)
        if atoms:
            from titan_b200.ops.mxfp8_gemm import pack_scale_atoms

            s1 = pack_scale_atoms(s1) if rows else None
            s2t = pack_scale_atoms(s2t) if transposed else None
        return q1, s1, q2t, s2t
    if not x.is_meta:
        _declare()
    x = x.contiguous()
    R, C = x.shape
    u8 = dict(dtype=torch.uint8, device=x.device)
    q1 = torch.empty(R, C, **u8) if rows else None
    q2t = torch.empty(C, R, **u8) if transposed else None
    if atoms:
        s1 = torch.empty(R // 128, C // 128, 512, **u8) if rows else None
        s2t = torch.empty(C // 128, R // 128, 512, **u8) if transposed else None
    else:
        s1 = torch.empty(R, C // BLOCK, **u8) if rows else None
        s2t = torch.empty(C, R // BLOCK, **u8) if transposed else None
    f8 = lambda t: t.view(torch.float8_e4m3fn) if t is not None else None  # noqa: E731
    if x.is_meta:   # shapes only (memory simulation)
        _lib.note_skipped_launch("tb_mx_quantize_dual", (None, None, None, None, None, R, C))
        return f8(q1), s1, f8(q2t), s2t
    p = lambda t: t.data_ptr() if t is not None else None  # noqa: E731
    rc = _lib.lib().tb_mx_quantize_dual(x.data_ptr(), p(q1), p(s1), p(q2t), p(s2t), R, C,
                                        {"floor": 0, "rceil": 1}[round_mode], _lib.dtype_code(x.dtype), int(atoms),
                                        _lib.stream_ptr())
    _lib.check(rc, "mx_quantize_dual")
    return f8(q1), s1, f8(q2t), s2t


def mx_dequantize(q: torch.Tensor, scales: torch.Tensor, axis: int = -1, dtype=torch.bfloat16):
    if not ((q.is_cuda or q.is_meta) and q.dim() == 2 and q.is_contiguous() and dtype == torch.bfloat16
            and q.shape[1] % 8 == 0):
        return mx_dequantize_ref(q, scales, axis, dtype)
    rows, cols = q.shape
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device=q.device)
    if q.is_meta:   # shapes only (memory simulation)
        _lib.note_skipped_launch("tb_mx_dequantize", (None, None, None, rows, cols))
        return out
    _declare()
    rc = _lib.lib().tb_mx_dequantize(q.view(torch.uint8).data_ptr(), scales.contiguous().data_ptr(), out.data_ptr(),
                                     rows, cols, axis, _lib.stream_ptr())
    _lib.check(rc, "mx_dequantize")
    return out


def mx_fake_quantize(x: torch.Tensor, axis: int = -1, round_mode: str = "rceil") -> torch.Tensor:
    """Quantise and dequantise: the value an MX GEMM would see, in x's dtype (no gradient logic here)."""
    if x.dim() == 2 and _kernel_ok(x, axis):
        q, s = mx_quantize(x, axis, round_mode)
        return mx_dequantize(q, s, axis).to(x.dtype)
    q, s = mx_quantize_ref(x, axis, round_mode)
    return mx_dequantize_ref(q, s, axis, x.dtype)


def sqnr(ref: torch.Tensor, test: torch.Tensor) -> float:
    """Signal-to-quantisation-noise ratio in dB."""
    ref, test = ref.detach().float(), test.detach().float()
    return float(10 * torch.log10(ref.pow(2).sum() / (ref - test).pow(2).sum().clamp_min(1e-30)))
