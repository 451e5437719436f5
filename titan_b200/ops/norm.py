"""RMSNorm: sm_100a kernel with autograd + the PyTorch oracle.

``rms_norm(x, w, eps)`` dispatches on the device of `x`: CUDA tensors run
`csrc/elementwise/rmsnorm.cu`; CPU tensors run the oracle (so recipes with the
converter switched on still run in CPU dry-run mode).

Parity: reference op `npu_rms_norm(x, w, eps)[0]` with rstd kept for backward
(torchtitan_npu/converters/kernels/rms_norm.py:39-44).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from titan_b200.ops import _lib

__all__ = ["rms_norm", "rms_norm_ref", "rms_norm_fwd", "rms_norm_bwd"]


def rms_norm_ref(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 oracle."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


def rms_norm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float):
    """→ (y, rstd[rows] fp32).  `x` is [..., dim] contiguous."""
    dim = x.shape[-1]
    x2 = x.reshape(-1, dim)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    if w.dtype != x.dtype:
        w = w.to(x.dtype)
    rc = _lib.lib().tb_rmsnorm_fwd(x2.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, dim, float(eps),
                                   _lib.dtype_code(x.dtype), _lib.stream_ptr())
    _lib.check(rc, "rmsnorm_fwd")
    return y.view(x.shape), rstd


def rms_norm_bwd(g: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor):
    """→ (dx, dw)."""
    dim = x.shape[-1]
    g2 = g.reshape(-1, dim).contiguous()
    x2 = x.reshape(-1, dim)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    rows = x2.shape[0]
    L = _lib.lib()
    grid = L.tb_rmsnorm_bwd_grid(rows, dim)
    scratch = torch.empty(grid * dim, dtype=torch.float32, device=x.device)
    dx = torch.empty_like(x2)
    wk = w if w.dtype == x.dtype else w.to(x.dtype)
    dw = torch.empty(dim, dtype=x.dtype, device=x.device)
    rc = L.tb_rmsnorm_bwd(g2.data_ptr(), x2.data_ptr(), wk.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                          scratch.data_ptr(), rows, dim, _lib.dtype_code(x.dtype), _lib.stream_ptr())
    _lib.check(rc, "rmsnorm_bwd")
    return dx.view(x.shape), dw.to(w.dtype)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        from titan_b200.ops.registry import ops

        y, rstd = ops.rms_norm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, g):
        from titan_b200.ops.registry import ops

        x, w, rstd = ctx.saved_tensors
        dx, dw = ops.rms_norm_bwd(g, x, w, rstd)
        return dx, dw, None


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    if x.is_cuda or x.is_meta:  # meta tensors take the operator's fake kernel (shapes and saved tensors as on a GPU)
        return _RMSNormFn.apply(x, w, eps)
    return F.rms_norm(x, (x.shape[-1],), w, eps)
