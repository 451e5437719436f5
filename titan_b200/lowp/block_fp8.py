"""Block-scaled FP8 linear: activations in 1×32 MX blocks, the WEIGHT in 32×32 blocks with one power-of-two scale each.

A 32×32 weight block is quantised ONCE and serves both GEMMs that read the weight: the forward contracts over K and
reads the block scale as the scale of 32 consecutive rows' K-block; the input gradient contracts over N and reads the
same byte as the scale of 32 consecutive columns' N-block.  Both are plain 1×32 scale operands of the block-scaled
tensor-core GEMM (`ops/mxfp8_gemm.py`), obtained by repeating the block scale 32 times along the other axis:

    forward  y  = mx(x, K) · blk(w)ᵀ                 scales of w: s[N/32, K/32] repeated down 32 rows     → [N, K/32]
    dgrad    dx = mx(g, N) · blk(w)                  scales of wᵀ: sᵀ[K/32, N/32] repeated down 32 rows   → [K, N/32]
    wgrad    dw = mx(gᵀ, T) · mx(xᵀ, T)ᵀ             both blocked down the token rows (dual-axis quantiser)

`mxfp4_prepass=True` first snaps the weight to the MXFP4 grid (e2m1 elements, 1×32 e8m0 scales), the nested
fake-quantiser of the reference's block configuration; the straight-through gradient reaches the original weight.

On the CPU, and for shapes the kernel does not take, the same quantised values go through dequantise + matmul.

Parity: `_BlockFP8QuantMM` / `to_block_fp8_then_mm` (experiments/ao_npu/torchao_npu/ops/block_ops.py),
`quantize_right_operand` (quantization/quant_primitives/block_fp8.py:19-42), `BlockQuantizeConfig`
(quantization/quant_configs.py:63-104).
"""

from __future__ import annotations

import torch

from titan_b200.lowp.mx import BLOCK, mx_dequantize_ref, mx_quantize_dual

__all__ = ["block_quantize_weight", "block_dequantize_weight", "block_fp8_linear", "block_fp8_grouped_mm", "BlockFP8MM"]

E4M3_MAX = 448.0


def block_quantize_weight(w: torch.Tensor, block: int = BLOCK):
    """w [..., N, K] (N, K multiples of ``block``) → (q float8_e4m3fn [..., N, K], s uint8 [..., N/block, K/block]);
    ``s`` is the e8m0 byte of the smallest power of two that keeps the block maximum within ±448."""
    *lead, N, K = w.shape
    if N % block or K % block:
        raise ValueError(f"block_quantize_weight: dims {N}x{K} must be multiples of {block}")
    tiles = w.float().reshape(*lead, N // block, block, K // block, block)
    amax = tiles.abs().amax(dim=(-3, -1))
    safe = amax.clamp_min(torch.finfo(torch.float32).tiny)
    e = torch.ceil(torch.log2(safe / E4M3_MAX))
    e = torch.where(safe * torch.exp2(-(e - 1)) <= E4M3_MAX, e - 1, e).clamp(-127, 127)
    e = torch.where(amax > 0, e, torch.full_like(e, -127))
    q = (tiles * torch.exp2(-e)[..., :, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(*lead, N, K), (e + 127).to(torch.uint8)


def block_dequantize_weight(q: torch.Tensor, s: torch.Tensor, block: int = BLOCK, dtype=torch.bfloat16) -> torch.Tensor:
    scale = torch.exp2(s.float() - 127.0).repeat_interleave(block, -1).repeat_interleave(block, -2)
    return (q.float() * scale).to(dtype)


def _rows_scales(s: torch.Tensor, block: int = BLOCK) -> torch.Tensor:
    """[R/32, C/32] block scales → [R, C/32]: the 1×32 scale operand of a GEMM contracting over C."""
    return s.repeat_interleave(block, dim=-2).contiguous()


def _gemm_q(aq, sa, bq, sb, dtype):
    if aq.is_cuda:
        from titan_b200.ops.mxfp8_gemm import mxfp8_gemm, mxfp8_gemm_supported

        if mxfp8_gemm_supported(aq.shape[0], bq.shape[0], aq.shape[1]):
            return mxfp8_gemm(aq, sa, bq, sb).to(dtype)
    return mx_dequantize_ref(aq, sa, -1, dtype) @ mx_dequantize_ref(bq, sb, -1, dtype).t()


class BlockFP8MM(torch.autograd.Function):
    """x [T, K] · w [N, K]ᵀ with T, N, K multiples of 32.  Saves the token-blocked fp8 copy of ``x`` and the quantised
    weight (1 byte per element each) instead of bf16 tensors."""

    @staticmethod
    def forward(ctx, x, w, round_mode: str = "rceil", mxfp4_prepass: bool = False):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype == torch.float32 and x2.is_cuda:
            x2 = x2.to(torch.bfloat16)
        dt = x2.dtype
        if mxfp4_prepass:
            from titan_b200.lowp.qat import mxfp4_fake_quantize

            w = mxfp4_fake_quantize(w)
        wq, ws = block_quantize_weight(w.to(dt))
        xq1, xs1, xq2t, xs2t = mx_quantize_dual(x2.contiguous(), round_mode, transposed=ctx.needs_input_grad[1])
        y = _gemm_q(xq1, xs1, wq, _rows_scales(ws), dt)
        ctx.save_for_backward(xq2t, xs2t, wq, ws)
        ctx.meta = (x.shape, x.dtype, w.dtype, dt, round_mode)
        return y.to(x.dtype).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, g):
        xq2t, xs2t, wq, ws = ctx.saved_tensors
        shape, x_dt, w_dt, dt, rm = ctx.meta
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        g2 = g.reshape(-1, g.shape[-1]).to(dt).contiguous()
        gq1, gs1, gq2t, gs2t = mx_quantize_dual(g2, rm, rows=need_dx, transposed=need_dw)
        dx = dw = None
        if need_dx:  # the SAME quantised weight, read transposed: byte transpose + transposed block scales
            wqt = wq.view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn)
            dx = _gemm_q(gq1, gs1, wqt, _rows_scales(ws.t()), dt).to(x_dt).reshape(shape)
        if need_dw:
            dw = _gemm_q(gq2t, gs2t, xq2t, xs2t, dt).to(w_dt)
        return dx, dw, None, None


def _fits(*dims: int) -> bool:
    return all(d > 0 and d % BLOCK == 0 for d in dims)


def block_fp8_linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, *,
                     round_mode: str = "rceil", mxfp4_prepass: bool = False) -> torch.Tensor:
    """`F.linear` through `BlockFP8MM`; the bias is added after the product.  Shapes with a dim that is not a multiple of
    32 (and empty inputs) fall back to the quantise-dequantise statement of the same arithmetic."""
    T = x.numel() // max(x.shape[-1], 1)
    if _fits(T, x.shape[-1], weight.shape[0]):
        y = BlockFP8MM.apply(x, weight, round_mode, mxfp4_prepass)
    else:
        from titan_b200.lowp.qat import QuantizeConfig, _STE

        wq = _STE.apply(weight, QuantizeConfig(kind="block_fp8", mxfp4_prepass=mxfp4_prepass))
        xq = _STE.apply(x, QuantizeConfig(kind="mx", round_mode=round_mode))
        y = xq @ wq.to(xq.dtype).t()
    return y if bias is None else y + bias


def block_fp8_grouped_mm(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor, *, round_mode: str = "rceil",
                         mxfp4_prepass: bool = False) -> torch.Tensor:
    """Grouped form: rows ``[offs[e-1], offs[e])`` of ``x [T, K]`` go through ``w[e] [N, K]`` (each expert's weight in its
    own 32×32 blocks; token-axis blocks of wgrad never straddle two experts)."""
    out = x.new_zeros(x.shape[0], w.shape[1])
    start = 0
    for e, end in enumerate(offs.tolist()):
        if end > start:
            out[start:end] = block_fp8_linear(x[start:end], w[e], round_mode=round_mode, mxfp4_prepass=mxfp4_prepass)
        start = end
    return out
