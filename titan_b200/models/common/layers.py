"""Shared model building blocks (baseline PyTorch math).

These are the library-op definitions every model is assembled from; the
fused sm_100a kernels replace them through model converters, never by editing
model code.

Parity: the reference assembles its models from upstream
`models.common.{Embedding, Linear, RMSNorm, FeedForward, ScaledDotProductAttention}`
(torchtitan_npu/models/deepseek_v4/moe.py:12-18, converters/kernels/rms_norm.py:39-44).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from titan_b200.protocols.module import Module

__all__ = ["Linear", "Embedding", "RMSNorm", "LayerNorm", "FeedForward", "ScaledDotProductAttention", "repeat_kv"]


class Linear(nn.Linear, Module):
    """`nn.Linear` with truncated-normal init controlled by ``init_std``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, init_std: float = 0.02,
                 device=None, dtype=None):
        nn.Linear.__init__(self, in_features, out_features, bias=bias, device=device, dtype=dtype)
        self.init_std = init_std

    def init_states(self, *, init_std: float | None = None, **kwargs) -> None:
        std = getattr(self, "init_std", 0.02) if init_std is None else init_std
        nn.init.trunc_normal_(self.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def reset_parameters(self) -> None:
        if self.weight.device.type != "meta":
            self.init_states()


class Embedding(nn.Embedding, Module):
    def init_states(self, **kwargs) -> None:
        nn.init.normal_(self.weight)

    def reset_parameters(self) -> None:
        if self.weight.device.type != "meta":
            self.init_states()


class RMSNorm(Module):
    """y = x * rsqrt(mean(x^2) + eps) * w, statistics in fp32."""

    def __init__(self, dim: int, eps: float | None = 1e-6, device=None, dtype=None):
        super().__init__()
        self.dim = dim
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        eps = self.eps if self.eps is not None else torch.finfo(x.dtype).eps
        w = self.weight
        if hasattr(w, "to_local") and not hasattr(x, "to_local"):
            # replicated weight on per-rank activations (local heads / sequence slice)
            from titan_b200.parallel.tensor_parallel import norm_weight_local

            w = norm_weight_local(w, x)
        return F.rms_norm(x, (self.dim,), w, eps)

    def init_states(self, **kwargs) -> None:
        nn.init.ones_(self.weight)

    def reset_parameters(self) -> None:
        if self.weight.device.type != "meta":
            self.init_states()


class LayerNorm(nn.LayerNorm, Module):
    def init_states(self, **kwargs) -> None:
        nn.LayerNorm.reset_parameters(self)


class FeedForward(Module):
    """SwiGLU MLP: w2(silu(w1 x) * w3 x)."""

    @dataclass(kw_only=True)
    class Config(Module.Config):
        dim: int = 256
        hidden_dim: int = 768

    def __init__(self, config: "FeedForward.Config | None" = None, *, dim: int | None = None,
                 hidden_dim: int | None = None):
        super().__init__()
        if config is not None:
            dim, hidden_dim = config.dim, config.hidden_dim
        self.w1 = Linear(dim, hidden_dim, bias=False)
        self.w2 = Linear(hidden_dim, dim, bias=False)
        self.w3 = Linear(dim, hidden_dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        limit = float(getattr(self, "swiglu_limit", 0.0) or 0.0)
        if limit > 0:  # DeepSeek-V4 clamps gate and up before the activation (models/deepseek_v4/moe.py:183-203)
            return self.w2(F.silu(self.w1(x).clamp(max=limit)) * self.w3(x).clamp(min=-limit, max=limit))
        return self.w2(F.silu(self.w1(x)) * self.w3(x))

    def init_states(self, *, init_std: float = 0.02, **kwargs) -> None:
        self.w1.init_states(init_std=0.02)
        self.w2.init_states(init_std=init_std)
        self.w3.init_states(init_std=init_std)


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[B, S, Hkv, D] → [B, S, Hkv*n_rep, D] (GQA expansion)."""
    if n_rep == 1:
        return x
    b, s, h, d = x.shape
    return x[:, :, :, None, :].expand(b, s, h, n_rep, d).reshape(b, s, h * n_rep, d)


class ScaledDotProductAttention(Module):
    """Library attention over [B, H, S, D] tensors (the baseline the fused kernel is compared with)."""

    def __init__(self, causal: bool = True):
        super().__init__()
        self.causal = causal

    def forward(self, q, k, v, *, scale: float | None = None, attn_mask: torch.Tensor | None = None):
        enable_gqa = q.shape[1] != k.shape[1]
        if attn_mask is not None:
            return F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, scale=scale, enable_gqa=enable_gqa)
        if q.is_cuda:
            # backend order of the upstream attention wrapper: the cuDNN kernel first (on B200 it runs the Llama-3 8B
            # shape at 1.38 PFLOP/s forward against 0.35 for the sm_80-style flash kernel), then flash, then the rest
            with _sdpa_backends():
                return F.scaled_dot_product_attention(q, k, v, is_causal=self.causal, scale=scale,
                                                      enable_gqa=enable_gqa)
        return F.scaled_dot_product_attention(q, k, v, is_causal=self.causal, scale=scale, enable_gqa=enable_gqa)


def _sdpa_backends():
    from torch.nn.attention import SDPBackend, sdpa_kernel

    return sdpa_kernel([SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION,
                        SDPBackend.MATH], set_priority=True)
