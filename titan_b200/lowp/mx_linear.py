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

Quantise once.  When every dim is a multiple of 32, `MXFP8MM` reads each operand once per pass with the dual-axis
kernel (`mx_quantize_dual`): the forward quantises ``x`` along K for its own GEMM and down the token rows, transposed,
for wgrad, and saves ONLY that fp8 copy (1 byte + 1/32 per element instead of the bf16 activation: half the saved
bytes, and no bf16 transpose in backward); the backward quantises ``g`` once into both views and the weight once into
its transposed view.  The weight is saved by reference rather than as a second quantised copy, so an FSDP-sharded
weight costs no unsharded bytes between forward and backward.  Parity for this form: `_MXQuantMM`
(experiments/ao_npu/torchao_npu/ops/mx_ops.py:62-194), which saves quantised copies of both operands.

Parity: `NpuMXFP8MM` (torchtitan_npu/patches/torchao_npu/mx_linear.py:26-100) and `NpuMXFP8GroupedMM`
(patches/torchao_npu/mxfp8_grouped_mm.py:22-170).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from titan_b200.lowp.mx import BLOCK, mx_dequantize, mx_fake_quantize, mx_quantize, mx_quantize_dual

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
    if (a.is_cuda or a.is_meta) and a.dtype == torch.bfloat16 and b_t.dtype == torch.bfloat16:
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


def _gemm_q(aq, sa, bq, sb, dtype) -> torch.Tensor:
    """``dequant(aq, sa) · dequant(bq, sb)ᵀ`` for operands already quantised along their shared last dim."""
    if aq.is_cuda or aq.is_meta:
        from titan_b200.ops.mxfp8_gemm import mxfp8_gemm, mxfp8_gemm_supported

        if sa.dim() == 3:  # scales already in the GEMM's atom order (only produced for shapes the kernel takes)
            return mxfp8_gemm(aq, sa, bq, sb, packed=True).to(dtype)
        if mxfp8_gemm_supported(aq.shape[0], bq.shape[0], aq.shape[1]):
            return mxfp8_gemm(aq, sa, bq, sb).to(dtype)
    return _mm(mx_dequantize(aq, sa, -1, dtype), mx_dequantize(bq, sb, -1, dtype))


def _once_ok(*dims: int) -> bool:
    return all(d > 0 and d % BLOCK == 0 for d in dims)


def _atoms_ok(t: torch.Tensor, *dims: int) -> bool:
    """The quantiser can emit the GEMM's scale layout directly: CUDA 16-bit input, every dim a multiple of 128."""
    return (t.is_cuda or t.is_meta) and t.dtype in (torch.bfloat16, torch.float16) and all(d % 128 == 0 for d in dims)


def _mx_linear_fwd(x2, w, round_mode: str, need_wgrad: bool, atoms: bool):
    """x2 [M, K], w [N, K] (16-bit, block-aligned) → (y [M, N], fp8 copy of x blocked down the token rows and its
    scales, kept for the weight gradient; empty when not needed).  One dispatcher operator
    (`titan_b200::mx_linear_fwd`), so selective checkpointing keeps its outputs instead of quantising and multiplying
    again in backward."""
    xq1, xs1, xq2t, xs2t = mx_quantize_dual(x2.contiguous(), round_mode, transposed=need_wgrad, atoms=atoms)
    wq1, ws1, _, _ = mx_quantize_dual(w.contiguous(), round_mode, transposed=False, atoms=atoms)
    y = _gemm_q(xq1, xs1, wq1, ws1, x2.dtype)
    if not need_wgrad:
        return y, x2.new_empty((0,), dtype=torch.float8_e4m3fn), x2.new_empty((0,), dtype=torch.uint8)
    return y, xq2t, xs2t


class MXFP8MM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, round_mode: str = "rceil"):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype == torch.float32 and (x2.is_cuda or x2.is_meta):
            x2 = x2.to(torch.bfloat16)
        wq = w.to(x2.dtype)
        ctx.meta = (x.shape, x.dtype, w.dtype, round_mode)
        ctx.once = _once_ok(x2.shape[0], x2.shape[1], w.shape[0])
        if ctx.once:
            ctx.atoms = at = _atoms_ok(x2, x2.shape[0], x2.shape[1], w.shape[0])
            if x2.is_cuda or x2.is_meta:
                from titan_b200.ops.registry import ops

                y, xq2t, xs2t = ops.mx_linear_fwd(x2, wq, round_mode, bool(ctx.needs_input_grad[1]), at)
            else:
                y, xq2t, xs2t = _mx_linear_fwd(x2, wq, round_mode, bool(ctx.needs_input_grad[1]), at)
            ctx.compute_dtype = x2.dtype
            ctx.save_for_backward(xq2t, xs2t, wq)
        else:
            y = _mm_mx(x2, wq, round_mode)
            ctx.save_for_backward(x2, wq)
        return y.to(x.dtype).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, g):
        shape, x_dt, w_dt, rm = ctx.meta
        if ctx.once:
            xq2t, xs2t, w = ctx.saved_tensors
            dt = ctx.compute_dtype
            need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
            g2 = g.reshape(-1, g.shape[-1]).to(dt).contiguous()
            gq1, gs1, gq2t, gs2t = mx_quantize_dual(g2, rm, rows=need_dx, transposed=need_dw, atoms=ctx.atoms)
            dx = dw = None
            if need_dx:  # dx = g · w: contraction over N, the weight blocked down its N rows and read transposed
                _, _, wq2t, ws2t = mx_quantize_dual(w.contiguous(), rm, rows=False, atoms=ctx.atoms)
                dx = _gemm_q(gq1, gs1, wq2t, ws2t, dt).to(x_dt).reshape(shape)
            if need_dw:  # dw = gᵀ · x: contraction over tokens, both operands blocked down the token rows
                dw = _gemm_q(gq2t, gs2t, xq2t, xs2t, dt).to(w_dt)
            return dx, dw, None
        x2, w = ctx.saved_tensors
        g2 = g.reshape(-1, g.shape[-1]).to(x2.dtype)
        # dx = g · w: contraction over N → g blocked along its rows' N, w blocked down its N rows
        dx = _mm_mx(g2, w.t().contiguous(), rm)
        # dw = gᵀ · x: contraction over tokens → both blocked down the token rows
        dw = _mm_mx(g2.t().contiguous(), x2.t().contiguous(), rm)
        return dx.to(x_dt).reshape(shape), dw.to(w_dt), None


def mx_linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, round_mode: str = "rceil"):
    y = MXFP8MM.apply(x, weight, round_mode)
    return y if bias is None else y + bias


# ---- quantised expert weights, kept between the optimizer steps
# Expert weights change once per optimizer step but are multiplied several times in between (forward, recomputed
# forward under activation checkpointing, input gradient; every micro-batch of a gradient-accumulation step).  A module
# that passes a `weight_key` gets both quantised views of its weight (row-blocked for the forward, transposed for the
# input gradient) from ONE dual-axis pass, kept until `invalidate_weight_cache()` (the optimizer containers call it
# after every step) or until the tensor's version counter moves (in-place loads).  Modules whose weight is resharded
# between uses (FSDP) must not pass a key: the cache would pin the unsharded bytes.
_WEIGHT_CACHE: dict = {}


def invalidate_weight_cache() -> None:
    _WEIGHT_CACHE.clear()


def _quantized_weight(w2d: torch.Tensor, round_mode: str, weight_key):
    """→ (wq, ws, wq_t, ws_t): row-blocked and transposed MX views of ``w2d`` [E*N, K], atom-ordered scales."""
    if weight_key is None:
        return None
    tag = (w2d._version, tuple(w2d.shape), w2d.data_ptr(), round_mode)
    hit = _WEIGHT_CACHE.get(weight_key)
    if hit is not None and hit[0] == tag:
        return hit[1]
    with torch.no_grad():
        views = mx_quantize_dual(w2d.contiguous(), round_mode, rows=True, transposed=True, atoms=True)
    _WEIGHT_CACHE[weight_key] = (tag, views)
    return views


class _MXGroupedMMAligned(torch.autograd.Function):
    """Grouped MXFP8 product over rows whose groups are multiples of 128 (the padded expert-major layout): three
    launches of the grouped block-scaled GEMM, operands quantised once each by the dual-axis kernel, no host sync.
    x [T, K], w [E, N, K], offs int32 [E] on the device → [T, N]; rows past the last group come back as zeros.  The
    buffer may have a ragged tail (capacity that is not a multiple of 128): the last group ends on a multiple of 128, so
    those rows are never routed to and only need a defined value."""

    @staticmethod
    def forward(ctx, x, w, offs, round_mode, weight_key=None):
        from titan_b200.ops.mxfp8_gemm import GROUP_B_ROWS, mxfp8_grouped_gemm

        E, N, K = w.shape
        T = x.shape[0]
        used = T // 128 * 128
        xq1, xs1, xq2t, xs2t = mx_quantize_dual(x[:used].contiguous(), round_mode, transposed=ctx.needs_input_grad[1],
                                                atoms=True)
        cached = _quantized_weight(w.reshape(E * N, K), round_mode, weight_key)
        if cached is not None:
            wq1, ws1 = cached[0], cached[1]
        else:
            wq1, ws1, _, _ = mx_quantize_dual(w.reshape(E * N, K).contiguous(), round_mode, transposed=False,
                                              atoms=True)
        ctx.save_for_backward(xq2t, xs2t, w, offs)
        ctx.round_mode, ctx.rows, ctx.weight_key = round_mode, T, weight_key
        y = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
        if used < T:
            y[used:].zero_()
        return mxfp8_grouped_gemm(xq1, xs1, wq1, ws1, offs, GROUP_B_ROWS, out=y, packed=True)

    @staticmethod
    def backward(ctx, g):
        from titan_b200.ops.mxfp8_gemm import GROUP_B_SLICE, GROUP_K, mxfp8_grouped_gemm

        xq2t, xs2t, w, offs = ctx.saved_tensors
        E, N, K = w.shape
        T = ctx.rows
        used = T // 128 * 128
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gq1, gs1, gq2t, gs2t = mx_quantize_dual(g[:used].contiguous(), ctx.round_mode, rows=need_dx,
                                                transposed=need_dw, atoms=True)
        dx = dw = None
        if need_dx:  # every expert's weight blocked down its N rows, transposed in the same pass: [K, E*N]
            cached = _quantized_weight(w.reshape(E * N, K), ctx.round_mode, ctx.weight_key)
            if cached is not None:
                wq2t, ws2t = cached[2], cached[3]
            else:
                _, _, wq2t, ws2t = mx_quantize_dual(w.reshape(E * N, K).contiguous(), ctx.round_mode, rows=False,
                                                    atoms=True)
            dx = torch.empty(T, K, dtype=torch.bfloat16, device=g.device)
            if used < T:
                dx[used:].zero_()
            mxfp8_grouped_gemm(gq1, gs1, wq2t, ws2t, offs, GROUP_B_SLICE, out=dx, packed=True)
        if need_dw:  # gᵀ [N, T] · xᵀ [K, T]ᵀ over each expert's own rows → [E*N, K]
            dw = mxfp8_grouped_gemm(gq2t, gs2t, xq2t, xs2t, offs, GROUP_K, packed=True).view(E, N, K).to(w.dtype)
        return dx, dw, None, None, None


def _aligned_ok(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor) -> bool:
    return ((x.is_cuda or x.is_meta) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and (offs.is_cuda or offs.is_meta)
            and x.shape[0] >= 128 and w.shape[1] % 128 == 0 and w.shape[2] % 128 == 0)


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


def mx_grouped_mm(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor, round_mode: str = "rceil", *,
                  aligned: bool = False, weight_key=None) -> torch.Tensor:
    """Grouped MXFP8 GEMM: rows ``[offs[e-1], offs[e])`` of ``x`` go through ``w[e]ᵀ``.  ``aligned=True`` is the
    caller's promise that every group is a multiple of 128 rows (the padded expert-major layout): on CUDA that form runs
    as one grouped tensor-core launch per product instead of a loop over experts.  ``weight_key`` (any hashable that
    names the weight) keeps the weight's quantised views between optimizer steps (see `invalidate_weight_cache`)."""
    if (aligned or x.is_meta) and _aligned_ok(x, w, offs):   # meta: shapes only, the host loop would read offs
        return _MXGroupedMMAligned.apply(x, w, offs.to(torch.int32), round_mode, weight_key)
    return _MXGroupedMM.apply(x, w, offs, round_mode)
