"""Hadamard rotation of the last dim (`rotate_activation`): FWHT kernel on CUDA, butterflies in PyTorch elsewhere.

Parity: `rotate_activation` / `hadamard_transform_ref` (torchtitan_npu/models/deepseek_v4/model.py:90-112,
models/deepseek_v32/model.py): ``x @ H_n · n^-0.5``.
"""

from __future__ import annotations

import ctypes

import torch

from titan_b200.ops import _lib

__all__ = ["hadamard", "hadamard_ref"]

_DECLARED = False


def hadamard_ref(x: torch.Tensor, scale: float) -> torch.Tensor:
    n = x.shape[-1]
    out = x.reshape(-1, n).float()
    h = 1
    while h < n:
        out = out.view(-1, n // (2 * h), 2, h)
        a, b = out[:, :, 0, :], out[:, :, 1, :]
        out = torch.stack((a + b, a - b), dim=2).reshape(-1, n)
        h *= 2
    return (out * scale).to(x.dtype).reshape(x.shape)


class _HadamardFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale):
        ctx.scale = scale
        return _run(x, scale)

    @staticmethod
    def backward(ctx, g):
        return _run(g.contiguous(), ctx.scale), None  # H is symmetric


def _run(x: torch.Tensor, scale: float) -> torch.Tensor:
    global _DECLARED
    if x.is_meta:   # shapes only (memory simulation)
        return torch.empty_like(x.contiguous())
    if not _DECLARED:
        P = ctypes.c_void_p
        _lib.declare("tb_hadamard", [P, P, ctypes.c_longlong, ctypes.c_int, ctypes.c_float, ctypes.c_int, P])
        _DECLARED = True
    x = x.contiguous()
    y = torch.empty_like(x)
    n = x.shape[-1]
    rc = _lib.lib().tb_hadamard(x.data_ptr(), y.data_ptr(), x.numel() // n, n, float(scale), _lib.dtype_code(x.dtype),
                                _lib.stream_ptr())
    _lib.check(rc, "hadamard")
    return y


def hadamard(x: torch.Tensor, scale: float | None = None) -> torch.Tensor:
    """``x @ H_n · scale`` over the last dim (default scale ``n^-0.5``: an orthonormal rotation)."""
    n = x.shape[-1]
    scale = n ** -0.5 if scale is None else scale
    if (x.is_cuda or x.is_meta) and x.dtype in (torch.bfloat16, torch.float16) and n in (64, 128, 256, 512):
        return _HadamardFn.apply(x, scale)
    return hadamard_ref(x, scale)
