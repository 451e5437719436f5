"""Rotary embedding: sm_100a kernel with autograd + oracle entry points.

Accepted caches: a complex ``[S, D/2]`` cache (interleaved layout), its real view
``[S, D/2, 2]``, or a real ``[S, 2·D]`` ``cos | sin`` cache (half-rotate layout).  Caches are
converted to the kernel's fp32 layout once and memoised per cache tensor.

Parity: reference RoPE wrapper (torchtitan_npu/converters/kernels/rope.py:68-201): complex →
interleaved cos/sin, real fp32 cache, `inverse` through negated sin, batch-shared positions.
"""

from __future__ import annotations

import weakref

import torch

from titan_b200.models.common import rope as rope_ref
from titan_b200.ops import _lib

__all__ = ["rope_apply", "apply_rotary_emb_complex", "apply_rotary_emb_single_complex", "apply_rotary_emb_cos_sin"]

_CACHE: dict[int, tuple] = {}


def _kernel_cache(cache: torch.Tensor) -> torch.Tensor:
    """fp32 contiguous cache in kernel layout; memoised on (tensor identity, data pointer, version)."""
    key = id(cache)
    hit = _CACHE.get(key)
    if hit is not None and hit[0]() is cache and hit[1] == (cache.data_ptr(), cache._version):
        return hit[2]
    if cache.is_complex():
        out = torch.view_as_real(cache).to(torch.float32).contiguous()
    else:
        out = cache.to(torch.float32).contiguous()
    if len(_CACHE) > 64:  # entries of dead tensors
        for k in [k for k, v in _CACHE.items() if v[0]() is None]:
            del _CACHE[k]
    _CACHE[key] = (weakref.ref(cache), (cache.data_ptr(), cache._version), out)
    return out


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cache, positions, interleaved, inverse):
        ctx.interleaved, ctx.inverse = interleaved, inverse
        ctx.save_for_backward(cache, positions if positions is not None else torch.empty(0))
        ctx.has_pos = positions is not None
        from titan_b200.ops.registry import ops

        return ops.rope(x, cache, positions, interleaved, inverse)

    @staticmethod
    def backward(ctx, g):
        cache, pos = ctx.saved_tensors
        # the rotation is orthogonal: its transpose is the rotation by the negative angle
        from titan_b200.ops.registry import ops

        return ops.rope(g, cache, pos if ctx.has_pos else None, ctx.interleaved, not ctx.inverse), None, None, None, None


def _launch(x: torch.Tensor, cache: torch.Tensor, positions, interleaved: bool, inverse: bool) -> torch.Tensor:
    if x.dim() != 4:
        raise ValueError(f"rope expects [B, S, H, D], got {tuple(x.shape)}")
    x = x.contiguous()
    B, S, H, D = x.shape
    y = torch.empty_like(x)
    cache_rows = cache.shape[0]
    pos_ptr, bstride = None, 0
    if positions is not None:
        positions = positions.to(device=x.device, dtype=torch.int64).contiguous()
        if positions.dim() == 2 and positions.shape[0] > 1:
            bstride = S
        positions = positions.reshape(-1)
        pos_ptr = positions.data_ptr()
    status = _lib.shared_status()
    rc = _lib.lib().tb_rope(x.data_ptr(), y.data_ptr(), cache.data_ptr(), pos_ptr, bstride, B, S, H, D, cache_rows,
                            1 if interleaved else 0, 1 if inverse else 0, _lib.dtype_code(x.dtype), status.ptr,
                            _lib.stream_ptr())
    _lib.check(rc, "rope")
    return y


def rope_apply(x: torch.Tensor, cache: torch.Tensor, positions=None, *, interleaved: bool = True,
               inverse: bool = False) -> torch.Tensor:
    """Rotate `x` [B, S, H, D]; CUDA → kernel, CPU → oracle."""
    if not (x.is_cuda or x.is_meta):
        if interleaved:
            c = cache if cache.is_complex() else torch.view_as_complex(cache.float().reshape(cache.shape[0], -1, 2))
            return rope_ref.apply_rotary_emb_single_complex(x, c, positions, inverse=inverse)
        c = cache
        if inverse:
            d = x.shape[-1]
            c = torch.cat([cache[..., :d], -cache[..., d:]], dim=-1)
        return rope_ref.apply_rotary_emb_cos_sin(x, x, c, positions)[0]
    return _RopeFn.apply(x, _kernel_cache(cache), positions, interleaved, inverse)


# drop-in replacements for the functions in `titan_b200.models.common.rope`
def apply_rotary_emb_single_complex(x, freqs_cis, positions=None, inverse: bool = False):
    return rope_apply(x, freqs_cis, positions, interleaved=True, inverse=inverse)


def apply_rotary_emb_complex(xq, xk, freqs_cis, positions=None):
    return (rope_apply(xq, freqs_cis, positions, interleaved=True),
            rope_apply(xk, freqs_cis, positions, interleaved=True))


def apply_rotary_emb_cos_sin(xq, xk, rope_cache, positions=None):
    return (rope_apply(xq, rope_cache, positions, interleaved=False),
            rope_apply(xk, rope_cache, positions, interleaved=False))
