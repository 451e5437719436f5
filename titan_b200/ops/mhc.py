"""Manifold-constrained hyper-connections (mHC): the residual stream is ``hc`` parallel copies ``[.., hc, D]``.

* `hc_split_sinkhorn` – turn the ``(2 + hc)·hc`` mixing logits of a token into ``pre`` (how the streams are
  collapsed into the sub-layer input), ``post`` (how the sub-layer output is written back to each stream)
  and ``comb`` (an ``hc × hc`` stream-mixing matrix pushed towards doubly-stochastic by Sinkhorn
  normalisation: softmax over the last axis, one column pass, then ``iters - 1`` row+column passes).
* `hc_pre`  – RMS statistics of the flattened streams → mixing logits ``F.linear(x, fn)·rsqrt`` →
  split/Sinkhorn → ``y = Σ_m pre[m]·x[m]``.
* `hc_post` – ``out[n] = post[n]·y + Σ_m comb[m, n]·residual[m]``.
* `hc_head` – final collapse of the streams with sigmoid weights.

The functions here are the fp32 PyTorch statement of the math; on CUDA with bf16 streams `hc_pre` / `hc_post`
dispatch to the fused sm_100a kernels when the converters ``b200_mhc_pre`` / ``b200_mhc_post`` enabled them
(one pass over the streams instead of six).

Parity: `HcSplitSinkhorn`, `HcPre`, `HcPost`, `HcHead` (torchtitan_npu/models/deepseek_v4/model.py:986-1075,
1209-1250) and the fused `npu_mhc_pre` / `npu_mhc_post` (converters/kernels/mhc.py).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from titan_b200.ops import _lib

__all__ = ["hc_split_sinkhorn", "hc_pre", "hc_post", "hc_head", "hc_pre_ref", "hc_post_ref", "hc_head_ref", "set_fused"]

_FUSED = {"pre": False, "post": False}


def set_fused(*, pre: bool | None = None, post: bool | None = None) -> None:
    """Switch the CUDA kernels on (done by the mHC converters)."""
    if pre is not None:
        _FUSED["pre"] = bool(pre)
    if post is not None:
        _FUSED["post"] = bool(post)


def _local(p):
    """Replicated mixing parameters applied to sequence-sharded streams: every rank sees other tokens, so the
    parameter gradient is a partial sum over the mesh."""
    if hasattr(p, "to_local"):
        from titan_b200.parallel.tensor_parallel import replicated_param_local

        return replicated_param_local(p, partial_grad=True)
    return p


def hc_split_sinkhorn(mixes: torch.Tensor, hc_scale: torch.Tensor, hc_base: torch.Tensor, hc_mult: int = 4,
                      sinkhorn_iters: int = 20, eps: float = 1e-6):
    """mixes [.., (2+hc)·hc] fp32 → pre [.., hc], post [.., hc], comb [.., hc, hc]."""
    hc = hc_mult
    pre, post, comb = mixes.split([hc, hc, hc * hc], dim=-1)
    pre = torch.sigmoid(pre * hc_scale[0] + hc_base[:hc]) + eps
    post = 2 * torch.sigmoid(post * hc_scale[1] + hc_base[hc: 2 * hc])
    comb = comb.unflatten(-1, (hc, hc)) * hc_scale[2] + hc_base[2 * hc:].view(hc, hc)
    comb = comb.softmax(-1) + eps
    comb = comb / (comb.sum(-2, keepdim=True) + eps)
    for _ in range(sinkhorn_iters - 1):
        comb = comb / (comb.sum(-1, keepdim=True) + eps)
        comb = comb / (comb.sum(-2, keepdim=True) + eps)
    return pre, post, comb


def hc_pre_ref(x, hc_fn, hc_scale, hc_base, hc_mult: int = 4, sinkhorn_iters: int = 20, hc_eps: float = 1e-6,
               norm_eps: float = 1e-6):
    shape, dtype = x.shape, x.dtype
    xf = x.flatten(-2).float()
    rsqrt = torch.rsqrt(xf.square().mean(-1, keepdim=True) + norm_eps)
    mixes = F.linear(xf, hc_fn.float()) * rsqrt
    pre, post, comb = hc_split_sinkhorn(mixes, hc_scale.float(), hc_base.float(), hc_mult, sinkhorn_iters, hc_eps)
    y = torch.sum(pre.unsqueeze(-1) * xf.view(shape), dim=-2)
    return y.to(dtype), post, comb


def hc_post_ref(x, residual, post, comb):
    y = post.unsqueeze(-1) * x.unsqueeze(-2).float() + torch.sum(
        comb.unsqueeze(-1) * residual.unsqueeze(-2).float(), dim=-3)
    return y.to(x.dtype)


def hc_pre(x, hc_fn, hc_scale, hc_base, hc_mult: int = 4, sinkhorn_iters: int = 20, hc_eps: float = 1e-6,
           norm_eps: float = 1e-6):
    """x [.., hc, D] → (y [.., D] in x.dtype, post [.., hc] fp32, comb [.., hc, hc] fp32)."""
    hc_fn, hc_scale, hc_base = _local(hc_fn), _local(hc_scale), _local(hc_base)
    if _FUSED["pre"] and _lib.on_device(x) and x.dtype == torch.bfloat16 and hc_mult == 4 and x.shape[-1] % 8 == 0:
        from titan_b200.ops import mhc_cuda

        return mhc_cuda.mhc_pre(x, hc_fn, hc_scale, hc_base, sinkhorn_iters, hc_eps, norm_eps)
    return hc_pre_ref(x, hc_fn, hc_scale, hc_base, hc_mult, sinkhorn_iters, hc_eps, norm_eps)


def hc_post(x, residual, post, comb):
    """x [.., D], residual [.., hc, D], post [.., hc], comb [.., hc, hc] → [.., hc, D]."""
    if (_FUSED["post"] and _lib.on_device(x) and x.dtype == torch.bfloat16 and residual.shape[-2] == 4
            and x.shape[-1] % 8 == 0):
        from titan_b200.ops import mhc_cuda

        return mhc_cuda.mhc_post(x, residual, post, comb)
    return hc_post_ref(x, residual, post, comb)


def hc_head(x, head_fn, head_scale, head_base, hc_eps: float = 1e-6, norm_eps: float = 1e-6):
    """Collapse the streams: x [.., hc, D] → [.., D] with weights ``sigmoid(mix·scale + base) + eps``."""
    head_fn, head_scale, head_base = _local(head_fn), _local(head_scale), _local(head_base)
    if (_FUSED["pre"] and _lib.on_device(x) and x.dtype == torch.bfloat16 and x.shape[-2] == 4 and x.shape[-1] % 8 == 0
            and x.shape[-1] <= 8192):
        # the collapse is the "pre" third of `hc_pre` (same RMS, same sigmoid weights, same weighted sum) with no
        # post / comb outputs: run the fused kernel on parameters padded with zero rows (one Sinkhorn pass on zeros)
        from titan_b200.ops import mhc_cuda

        fn24 = torch.cat([head_fn.float(), head_fn.new_zeros(20, head_fn.shape[1], dtype=torch.float32)], dim=0)
        scale3 = torch.cat([head_scale.float().reshape(1), head_scale.new_zeros(2, dtype=torch.float32)])
        base24 = torch.cat([head_base.float(), head_base.new_zeros(20, dtype=torch.float32)])
        return mhc_cuda.mhc_pre(x, fn24, scale3, base24, 1, hc_eps, norm_eps)[0]
    return hc_head_ref(x, head_fn, head_scale, head_base, hc_eps, norm_eps)


def hc_head_ref(x, head_fn, head_scale, head_base, hc_eps: float = 1e-6, norm_eps: float = 1e-6):
    shape, dtype = x.shape, x.dtype
    xf = x.flatten(-2).float()
    rsqrt = torch.rsqrt(xf.square().mean(-1, keepdim=True) + norm_eps)
    mixes = F.linear(xf, head_fn.float()) * rsqrt
    pre = torch.sigmoid(mixes * head_scale.float() + head_base.float()) + hc_eps
    return torch.sum(pre.unsqueeze(-1) * xf.view(shape), dim=-2).to(dtype)
