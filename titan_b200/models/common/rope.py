"""Rotary position embeddings: cache builders and the three apply layouts.

* ``apply_rotary_emb_complex(xq, xk, freqs_cis)`` – interleaved pairs
  ``(x[2i], x[2i+1])`` rotated by a complex cache ``[S, D/2]`` (Llama, DeepSeek).
* ``apply_rotary_emb_single_complex(x, freqs_cis)`` – same for one tensor.
* ``apply_rotary_emb_cos_sin(xq, xk, rope_cache)`` – half-rotate layout with a
  real cache ``[S, 2·D]`` holding ``cos | sin`` (Qwen3).

`positions` (``[B, S]`` or ``[S]``) gathers cache rows for packed documents;
``inverse=True`` rotates by the negative angle (DeepSeek-V4 un-rotates the
attention output).

Parity: these are the functions the reference's RoPE converter replaces
(torchtitan_npu/converters/kernels/rope.py:32-281).
"""

from __future__ import annotations

import math

import torch

__all__ = [
    "precompute_freqs_cis",
    "precompute_rope_cache",
    "apply_rotary_emb_complex",
    "apply_rotary_emb_single_complex",
    "apply_rotary_emb_cos_sin",
    "reshape_for_broadcast",
    "yarn_inv_freq",
]


def _llama3_scale(freqs: torch.Tensor, scaling_factor: float, low_freq_factor: float, high_freq_factor: float,
                  original_max_pos: int) -> torch.Tensor:
    low_wavelen = original_max_pos / low_freq_factor
    high_wavelen = original_max_pos / high_freq_factor
    wavelen = 2 * math.pi / freqs
    smooth = (original_max_pos / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    scaled = torch.where(wavelen > low_wavelen, freqs / scaling_factor, freqs)
    mid = (1 - smooth) * freqs / scaling_factor + smooth * freqs
    is_mid = (wavelen <= low_wavelen) & (wavelen >= high_wavelen)
    return torch.where(is_mid, mid, scaled)


def yarn_inv_freq(dim: int, theta: float, factor: float, original_seq_len: int, beta_fast: float = 32,
                  beta_slow: float = 1) -> torch.Tensor:
    """YaRN-corrected inverse frequencies (DeepSeek long-context extension)."""
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))

    def corr_dim(num_rot):
        return dim * math.log(original_seq_len / (num_rot * 2 * math.pi)) / (2 * math.log(theta))

    low = max(math.floor(corr_dim(beta_fast)), 0)
    high = min(math.ceil(corr_dim(beta_slow)), dim - 1)
    if low == high:
        high += 0.001
    ramp = torch.clamp((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low), 0, 1)
    smooth = 1 - ramp
    return freqs / factor * (1 - smooth) + freqs * smooth


def precompute_freqs_cis(dim: int, end: int, theta: float = 10000.0, *, scaling: dict | None = None,
                         inv_freq: torch.Tensor | None = None, device=None) -> torch.Tensor:
    """Complex cache ``[end, dim/2]`` (complex64)."""
    if inv_freq is None:
        inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device)[: dim // 2].float() / dim))
        if scaling:
            inv_freq = _llama3_scale(inv_freq, **scaling)
    t = torch.arange(end, device=inv_freq.device, dtype=torch.float32)
    ang = torch.outer(t, inv_freq)
    return torch.polar(torch.ones_like(ang), ang)


def precompute_rope_cache(dim: int, end: int, theta: float = 1_000_000.0, device=None) -> torch.Tensor:
    """Real cache ``[end, 2*dim]`` = ``cos(angles ⊕ angles) | sin(angles ⊕ angles)`` (half-rotate layout)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device).float() / dim))
    t = torch.arange(end, device=inv_freq.device, dtype=torch.float32)
    ang = torch.outer(t, inv_freq)
    emb = torch.cat([ang, ang], dim=-1)
    return torch.cat([emb.cos(), emb.sin()], dim=-1)


def reshape_for_broadcast(cache: torch.Tensor, x: torch.Tensor, positions: torch.Tensor | None = None):
    """Bring a ``[S_max, F]`` cache to ``[1|B, S, 1, F]`` for ``x`` of shape ``[B, S, H, ·]``."""
    seqlen = x.shape[1]
    if positions is None:
        return cache[:seqlen].view(1, seqlen, 1, cache.shape[-1])
    if positions.dim() == 1:
        return cache[positions].view(1, seqlen, 1, cache.shape[-1])
    return cache[positions].view(positions.shape[0], seqlen, 1, cache.shape[-1])


def apply_rotary_emb_single_complex(x: torch.Tensor, freqs_cis: torch.Tensor, positions: torch.Tensor | None = None,
                                    inverse: bool = False) -> torch.Tensor:
    dtype = x.dtype
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    f = reshape_for_broadcast(freqs_cis, x, positions)
    if inverse:
        f = f.conj()
    return torch.view_as_real(xc * f).flatten(-2).to(dtype)


def apply_rotary_emb_complex(xq: torch.Tensor, xk: torch.Tensor, freqs_cis: torch.Tensor,
                             positions: torch.Tensor | None = None):
    return (
        apply_rotary_emb_single_complex(xq, freqs_cis, positions),
        apply_rotary_emb_single_complex(xk, freqs_cis, positions),
    )


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_emb_cos_sin(xq: torch.Tensor, xk: torch.Tensor, rope_cache: torch.Tensor,
                             positions: torch.Tensor | None = None):
    hd = xq.shape[-1]
    c = reshape_for_broadcast(rope_cache, xq, positions)
    cos, sin = c[..., :hd], c[..., hd:]
    q = (xq.float() * cos) + (_rotate_half(xq.float()) * sin)
    k = (xk.float() * cos) + (_rotate_half(xk.float()) * sin)
    return q.type_as(xq), k.type_as(xk)
