"""MXFP8 matmuls with autograd: every GEMM of forward, dgrad and wgrad sees BOTH operands quantised to MXFP8 with 1×32
blocks along ITS contraction dim, accumulation in fp32, bf16 output.

    forward  y  = mx(x, K) · mx(w, K)ᵀ            x [T, K], w [N, K]   blocks along K
    dgrad    dx = mx(g, N) · mx(w, N-axis)        g [T, N]: blocks along N; w blocks down its rows (axis −2)
    wgrad    dw = mx(g, T-axis)ᵀ · mx(x, T-axis)  both blocked down the token rows (axis −2)

On CUDA every such product whose shape the kernel takes (rows a multiple of 128, contraction a multiple of 128) runs as
ONE block-scaled FP8 GEMM (`ops/mxfp8_gemm.py`: ``tcgen05.mma kind::mxf8f6f4.block_scale`` with the e8m0 scales in
tensor memory, 2.2 PFLOP/s on 8192x4096x4096 against 1.6 for the bf16 library GEMM).  Other shapes, and the CPU, use the
same numbers through quantise-dequantise + a bf16 / fp32 matmul: the quantised operands are exact in bf16
(e4m3 × 2^e), accumulation is fp32 either way.  Grouped experts (`mx_grouped_mm`) quantise per group along the token
axis for wgrad.

Parity: `NpuMXFP8MM` (torchtitan_npu/patches/torchao_npu/mx_linear.py:26-100) and `NpuMXFP8GroupedMM`
(patches/torchao_npu/mxfp8_grouped_mm.py:22-170).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from titan_b200.lowp.mx import BLOCK, mx_fake_quantize, mx_quantize

__all__ = ["mx_linear", "mx_grouped_mm", "MXFP8MM"]


def _fq(t: torch.Tensor, axis: int, round_mode: str) -> torch.Tensor:
    """Quantise-dequantise ``t`` (2-D) along ``axis``; a ragged quantised dim is zero-padded to a block multiple."""
    dim = t.shape[axis]
    pad = (-dim) % BLOCK
    if pad:
        t = F.pad(t, (0, pad)) if axis == -1 else F.pad(t, (0, 0, 0, pad))
    out = mx_fake_quantize(t.contiguous(), axis, round_mode)
    if pad:
        out = out[..., :dim] if axis == -1 else out[:dim]
    return out


def _mm_mx(a: torch.Tensor, b_t: torch.Tensor, round_mode: str) -> torch.Tensor:
    """``mx(a, K) · mx(b_t, K)ᵀ`` for a [M, K], b_t [N, K], both quantised in 1×32 blocks along K."""
    if a.is_cuda and a.dtype == torch.bfloat16 and b_t.dtype == torch.bfloat16:
        from titan_b200.ops.mxfp8_gemm import mxfp8_gemm, mxfp8_gemm_supported

        if mxfp8_gemm_supported(a.shape[0], b_t.shape[0], a.shape[1]):
            aq, sa = mx_quantize(a.contiguous(), -1, round_mode)
            bq, sb = mx_quantize(b_t.contiguous(), -1, round_mode)
            return mxfp8_gemm(aq, sa, bq, sb)
    return _mm(_fq(a, -1, round_mode), _fq(b_t, -1, round_mode))


def _mm(a: torch.Tensor, b_t: torch.Tensor) -> torch.Tensor:
    """a [M, K] · b_tᵀ with b_t [N, K] → [M, N] (tcgen05 GEMM on CUDA bf16, library matmul otherwise)."""
    if a.is_cuda and a.dtype in (torch.bfloat16, torch.float16) and a.shape[1] % 8 == 0:
        from titan_b200.ops.gemm import gemm

        return gemm(a.contiguous(), b_t.contiguous())
    return a @ b_t.t()


class MXFP8MM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, round_mode: str = "rceil"):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype == torch.float32 and x2.is_cuda:
            x2 = x2.to(torch.bfloat16)
        wq = w.to(x2.dtype)
        y = _mm_mx(x2, wq, round_mode)
        ctx.save_for_backward(x2, wq)
        ctx.meta = (x.shape, x.dtype, w.dtype, round_mode)
        return y.to(x.dtype).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, g):
        x2, w = ctx.saved_tensors
        shape, x_dt, w_dt, rm = ctx.meta
        g2 = g.reshape(-1, g.shape[-1]).to(x2.dtype)
        # dx = g · w: contraction over N → g blocked along its rows' N, w blocked down its N rows
        dx = _mm_mx(g2, w.t().contiguous(), rm)
        # dw = gᵀ · x: contraction over tokens → both blocked down the token rows
        dw = _mm_mx(g2.t().contiguous(), x2.t().contiguous(), rm)
        return dx.to(x_dt).reshape(shape), dw.to(w_dt), None


def mx_linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, round_mode: str = "rceil"):
    y = MXFP8MM.apply(x, weight, round_mode)
    return y if bias is None else y + bias


class _MXGroupedMM(torch.autograd.Function):
    """x [T, K] rows grouped by expert (``offs`` = cumulative row ends), w [E, N, K] → [T, N]."""

    @staticmethod
    def forward(ctx, x, w, offs, round_mode):
        E = w.shape[0]
        ends = offs.tolist()
        out = x.new_zeros(x.shape[0], w.shape[1])
        start = 0
        for e in range(E):
            if ends[e] > start:
                out[start:ends[e]] = _mm_mx(x[start:ends[e]], w[e], round_mode)
            start = ends[e]
        ctx.save_for_backward(x, w, offs)
        ctx.round_mode = round_mode
        return out

    @staticmethod
    def backward(ctx, g):
        x, w, offs = ctx.saved_tensors
        rm = ctx.round_mode
        ends = offs.tolist()
        g = g.contiguous()
        dx = torch.zeros_like(x)
        dw = torch.zeros_like(w)
        start = 0
        for e in range(w.shape[0]):
            end = ends[e]
            if end > start:
                dx[start:end] = _mm_mx(g[start:end], w[e].t().contiguous(), rm)
                # per-group quantisation along the group's own token rows
                dw[e] = _mm_mx(g[start:end].t().contiguous(), x[start:end].t().contiguous(), rm)
            start = end
        return dx, dw, None, None


def mx_grouped_mm(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor, round_mode: str = "rceil") -> torch.Tensor:
    """Grouped MXFP8 GEMM: rows ``[offs[e-1], offs[e])`` of ``x`` go through ``w[e]ᵀ``."""
    return _MXGroupedMM.apply(x, w, offs, round_mode)
