"""CUDA path of the hyper-connection ops (bf16 streams, hc = 4): autograd functions around the kernels of
`csrc/elementwise/mhc.cu` and the tcgen05 GEMM.

`mhc_pre` forward:  raw = x_flat · [fn_hi; fn_lo]ᵀ on the tensor cores (fn is fp32: its bf16 hi/lo split keeps ~16
mantissa bits, the products with the bf16 activations are exact, accumulation is fp32), then ONE kernel per token
for RMS statistic, mixing logits, Sinkhorn and the weighted stream sum.
`mhc_pre` backward: one kernel for the four ``gy·x[m]`` dots and the whole small-matrix backward (sigmoid, 20 Sinkhorn
passes, softmax) → a [T, 64] bf16 operand ``G``; ``dxf = G · fn`` and ``dfn = Gᵀ · x_flat`` on the tensor cores; one
kernel assembles ``dx = pre·gy + coef·x + dxf``.  The gradients of ``scale`` / ``base`` are sums over tokens of
[T, 24] tensors.
`mhc_post`: one kernel forward, one backward (dy, dres and the 20 dot products for dpost / dcomb).

Parity: the fused `npu_mhc_pre` / `npu_mhc_post` of the reference (converters/kernels/mhc_prepost.py).
"""

from __future__ import annotations

import ctypes

import torch

from titan_b200.ops import _lib
from titan_b200.ops.gemm import gemm

__all__ = ["mhc_pre", "mhc_post"]

_P, _I, _LL, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_DECLARED = False


def _declare():
    global _DECLARED
    if _DECLARED:
        return
    _lib.declare("tb_mhc_pre_fwd", [_P, _P, _LL, _P, _P, _I, _F, _F, _LL, _I, _P, _P, _P, _P, _P, _P])
    _lib.declare("tb_mhc_pre_bwd_small", [_P, _P, _P, _LL, _P, _P, _P, _P, _P, _P, _I, _F, _LL, _I, _P, _P, _P, _P, _P])
    _lib.declare("tb_mhc_pre_bwd_dx", [_P, _P, _P, _P, _P, _LL, _I, _P, _P])
    _lib.declare("tb_mhc_post_fwd", [_P, _P, _P, _P, _LL, _I, _P, _P])
    _lib.declare("tb_mhc_post_bwd", [_P, _P, _P, _P, _P, _LL, _I, _P, _P, _P, _P, _P])
    _DECLARED = True


def _split_fn(fn: torch.Tensor) -> torch.Tensor:
    """fp32 [24, 4D] → bf16 [64, 4D]: rows 0..23 = hi, rows 32..55 = lo (fn ≈ hi + lo), the rest zero."""
    hi = fn.to(torch.bfloat16)
    lo = (fn - hi.float()).to(torch.bfloat16)
    out = torch.zeros(64, fn.shape[1], dtype=torch.bfloat16, device=fn.device)
    out[:24], out[32:56] = hi, lo
    return out


class _MHCPre(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, fn, scale, base, iters, hc_eps, norm_eps):
        _declare()
        shape = x.shape
        D = shape[-1]
        x2 = x.reshape(-1, 4 * D)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        fn64 = _split_fn(fn.detach().float())
        raw = gemm(x2, fn64, out_dtype=torch.float32)  # [T, 64]
        dev = x.device
        y = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
        post = torch.empty(T, 4, dtype=torch.float32, device=dev)
        comb = torch.empty(T, 16, dtype=torch.float32, device=dev)
        pre = torch.empty(T, 4, dtype=torch.float32, device=dev)
        rstd = torch.empty(T, dtype=torch.float32, device=dev)
        sc, bs = scale.detach().float().contiguous(), base.detach().float().contiguous()
        rc = _lib.lib().tb_mhc_pre_fwd(x2.data_ptr(), raw.data_ptr(), raw.stride(0), sc.data_ptr(), bs.data_ptr(),
                                       int(iters), float(hc_eps), float(norm_eps), T, D, y.data_ptr(),
                                       post.data_ptr(), comb.data_ptr(), pre.data_ptr(), rstd.data_ptr(),
                                       _lib.stream_ptr())
        _lib.check(rc, "mhc_pre_fwd")
        ctx.save_for_backward(x2, raw, sc, bs, pre, rstd, fn64)
        ctx.meta = (shape, int(iters), float(hc_eps), fn.dtype, scale.dtype, base.dtype)
        lead = shape[:-2]
        return y.view(*lead, D), post.view(*lead, 4), comb.view(*lead, 4, 4)

    @staticmethod
    def backward(ctx, gy, gpost, gcomb):
        x2, raw, sc, bs, pre, rstd, fn64 = ctx.saved_tensors
        shape, iters, hc_eps, fn_dt, sc_dt, bs_dt = ctx.meta
        T, D = x2.shape[0], shape[-1]
        dev = x2.device
        gy = (gy if gy is not None else torch.zeros(T, D, dtype=torch.bfloat16, device=dev))
        gy = gy.reshape(T, D).to(torch.bfloat16).contiguous()
        gpost = (gpost.reshape(T, 4).float() if gpost is not None else torch.zeros(T, 4, device=dev)).contiguous()
        gcomb = (gcomb.reshape(T, 16).float() if gcomb is not None else torch.zeros(T, 16, device=dev)).contiguous()
        dz = torch.empty(T, 24, dtype=torch.float32, device=dev)
        mixes = torch.empty(T, 24, dtype=torch.float32, device=dev)
        G = torch.empty(T, 64, dtype=torch.bfloat16, device=dev)
        coef = torch.empty(T, dtype=torch.float32, device=dev)
        L = _lib.lib()
        rc = L.tb_mhc_pre_bwd_small(x2.data_ptr(), gy.data_ptr(), raw.data_ptr(), raw.stride(0), sc.data_ptr(),
                                    bs.data_ptr(), rstd.data_ptr(), pre.data_ptr(), gpost.data_ptr(),
                                    gcomb.data_ptr(), iters, hc_eps, T, D, dz.data_ptr(), mixes.data_ptr(),
                                    G.data_ptr(), coef.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "mhc_pre_bwd_small")
        # dxf = G[:, :24] · fn: contraction over the 64 (padded) mixing rows, B stored [K, N]
        fn_kn = torch.zeros(64, 4 * D, dtype=torch.bfloat16, device=dev)
        fn_kn[:24] = fn64[:24]
        dxf = gemm(G, fn_kn, b_mn=True)  # [T, 4D] bf16
        dx = torch.empty(T, 4 * D, dtype=torch.bfloat16, device=dev)
        rc = L.tb_mhc_pre_bwd_dx(x2.data_ptr(), gy.data_ptr(), dxf.data_ptr(), pre.data_ptr(), coef.data_ptr(), T, D,
                                 dx.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "mhc_pre_bwd_dx")
        # dfn = Gᵀ · x_flat: both operands stored contraction-major ([T, 64] and [T, 4D])
        dfn = gemm(G, x2, a_mn=True, b_mn=True, out_dtype=torch.float32)[:24]
        dbase = dz.sum(0)
        prod = dz * mixes
        dscale = torch.stack([prod[:, :4].sum(), prod[:, 4:8].sum(), prod[:, 8:].sum()])
        return dx.view(shape), dfn.to(fn_dt), dscale.to(sc_dt), dbase.to(bs_dt), None, None, None


class _MHCPost(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, res, post, comb):
        _declare()
        D = y.shape[-1]
        y2 = y.reshape(-1, D).contiguous()
        r2 = res.reshape(-1, 4 * D).contiguous()
        T = y2.shape[0]
        p2, c2 = post.reshape(T, 4).float().contiguous(), comb.reshape(T, 16).float().contiguous()
        out = torch.empty(T, 4 * D, dtype=torch.bfloat16, device=y.device)
        rc = _lib.lib().tb_mhc_post_fwd(y2.data_ptr(), r2.data_ptr(), p2.data_ptr(), c2.data_ptr(), T, D,
                                        out.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "mhc_post_fwd")
        ctx.save_for_backward(y2, r2, p2, c2)
        ctx.meta = (res.shape, y.shape, post.shape, comb.shape, post.dtype, comb.dtype)
        return out.view(res.shape)

    @staticmethod
    def backward(ctx, go):
        y2, r2, p2, c2 = ctx.saved_tensors
        res_shape, y_shape, post_shape, comb_shape, p_dt, c_dt = ctx.meta
        T, D = y2.shape
        g2 = go.reshape(T, 4 * D).to(torch.bfloat16).contiguous()
        dev = go.device
        dy = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
        dres = torch.empty(T, 4 * D, dtype=torch.bfloat16, device=dev)
        dpost = torch.empty(T, 4, dtype=torch.float32, device=dev)
        dcomb = torch.empty(T, 16, dtype=torch.float32, device=dev)
        rc = _lib.lib().tb_mhc_post_bwd(g2.data_ptr(), y2.data_ptr(), r2.data_ptr(), p2.data_ptr(), c2.data_ptr(), T,
                                        D, dy.data_ptr(), dres.data_ptr(), dpost.data_ptr(), dcomb.data_ptr(),
                                        _lib.stream_ptr())
        _lib.check(rc, "mhc_post_bwd")
        return dy.view(y_shape), dres.view(res_shape), dpost.view(post_shape).to(p_dt), dcomb.view(comb_shape).to(c_dt)


def mhc_pre(x, hc_fn, hc_scale, hc_base, sinkhorn_iters: int = 20, hc_eps: float = 1e-6, norm_eps: float = 1e-6):
    """x [.., 4, D] bf16 → (y [.., D] bf16, post [.., 4] fp32, comb [.., 4, 4] fp32)."""
    if x.shape[-2] != 4 or x.dtype != torch.bfloat16 or x.shape[-1] % 8 or x.shape[-1] > 8192:
        raise _lib.KernelError(f"mhc_pre: needs bf16 [.., 4, D] with D % 8 == 0 and D <= 8192, got {tuple(x.shape)}")
    return _MHCPre.apply(x, hc_fn, hc_scale, hc_base, sinkhorn_iters, hc_eps, norm_eps)


def mhc_post(x, residual, post, comb):
    """x [.., D] bf16, residual [.., 4, D] bf16, post [.., 4], comb [.., 4, 4] → [.., 4, D] bf16."""
    if x.dtype != torch.bfloat16 or residual.dtype != torch.bfloat16 or residual.shape[-2] != 4:
        raise _lib.KernelError("mhc_post: needs bf16 x [.., D] and residual [.., 4, D]")
    return _MHCPost.apply(x, residual, post, comb)
