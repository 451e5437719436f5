"""Multi-tensor reductions over lists of gradient tensors (`csrc/elementwise/adamw.cu`, same chunk table as the fused
AdamW): `sum_of_squares(tensors)` = Σ_t Σ_i t_i² in fp32, a handful of launches for a whole model instead of one
per parameter.  Every 65536-element chunk yields one partial and the partials are summed in a fixed order, so the
result is reproducible from run to run.

Counterpart of `torch._foreach_norm` as used by gradient clipping (the reference clips through
`torch.nn.utils.clip_grad_norm_` semantics, torchtitan_npu/patches/distributed/utils.py)."""

from __future__ import annotations

import ctypes

import torch

from titan_b200.ops import _lib

__all__ = ["sum_of_squares", "sum_of_squares_supported"]

_CHUNK = 65536
_DECLARED = False


def sum_of_squares_supported(tensors) -> bool:
    return (len(tensors) > 0 and all(t.is_cuda and t.is_contiguous() for t in tensors)
            and tensors[0].dtype in (torch.float32, torch.bfloat16, torch.float16)
            and all(t.dtype == tensors[0].dtype and t.device == tensors[0].device for t in tensors))


def sum_of_squares(tensors: list[torch.Tensor]) -> torch.Tensor:
    """fp32 0-d tensor: the sum of the squares of all elements of all `tensors` (one dtype, one CUDA device)."""
    global _DECLARED
    if not _DECLARED:
        P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        _lib.declare("tb_multi_sumsq", [P, P, I, I, P, LL, P, P])
        _DECLARED = True
    tensors = [t for t in tensors if t.numel() > 0]
    if not tensors:
        return torch.zeros((), dtype=torch.float32)
    n = len(tensors)
    cap = sum((t.numel() + _CHUNK - 1) // _CHUNK for t in tensors)
    partials = torch.empty(cap, dtype=torch.float32, device=tensors[0].device)
    ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in tensors])
    numel = (ctypes.c_longlong * n)(*[t.numel() for t in tensors])
    written = ctypes.c_longlong(0)
    rc = _lib.lib().tb_multi_sumsq(ptrs, numel, n, _lib.dtype_code(tensors[0].dtype), partials.data_ptr(), cap,
                                   ctypes.byref(written), _lib.stream_ptr())
    _lib.check(rc, "multi_sumsq")
    return partials[: written.value].sum()
