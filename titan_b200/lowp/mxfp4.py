"""MXFP4 storage format: e2m1 elements (±{0, 0.5, 1, 1.5, 2, 3, 4, 6}) packed two per byte, one e8m0 scale per 32.

* `mxfp4_quantize(x)` → ``(packed uint8 [..., K/2], scales uint8 [..., K/32])``: element ``2i`` in the low nibble,
  ``2i+1`` in the high nibble; a nibble is ``sign << 3 | index into the magnitude grid``.  The block exponent is the
  smallest power of two that keeps the block maximum within ±6; ties between grid points round to the even index.
* `mxfp4_dequantize(packed, scales)` → bf16 through a 256-entry table holding the PAIR of values of every byte, so a
  byte becomes two outputs with one gather, then × 2^(scale − 127).

Parity: `mxfp4_dequantize` (experiments/ao_npu/torchao_npu/quantization/quant_primitives/mx.py:18-94).
"""

from __future__ import annotations

import torch

from titan_b200.lowp.mx import BLOCK

__all__ = ["mxfp4_quantize", "mxfp4_dequantize", "E2M1_GRID"]

E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_PAIR_LUT: dict[torch.device, torch.Tensor] = {}


def _pair_lut(device: torch.device) -> torch.Tensor:
    lut = _PAIR_LUT.get(device)
    if lut is None:
        grid = torch.tensor(E2M1_GRID)
        nib = torch.cat([grid, -grid])  # codes 0..7 positive, 8..15 negative
        codes = torch.arange(256)
        lut = torch.stack([nib[codes & 0xF], nib[codes >> 4]], dim=-1).to(device)  # [256, 2]: (low, high)
        _PAIR_LUT[device] = lut
    return lut


def mxfp4_quantize(x: torch.Tensor):
    K = x.shape[-1]
    if K % BLOCK:
        raise ValueError(f"mxfp4_quantize: the last dim ({K}) must be a multiple of {BLOCK}")
    blocks = x.float().reshape(*x.shape[:-1], K // BLOCK, BLOCK)
    amax = blocks.abs().amax(-1)
    safe = amax.clamp_min(torch.finfo(torch.float32).tiny)
    e = torch.ceil(torch.log2(safe / 6.0))
    e = torch.where(safe * torch.exp2(-(e - 1)) <= 6.0, e - 1, e).clamp(-127, 127)
    e = torch.where(amax > 0, e, torch.full_like(e, -127))
    v = blocks * torch.exp2(-e).unsqueeze(-1)
    grid = torch.tensor(E2M1_GRID, device=x.device)
    # nearest grid point; bucketize on the midpoints sends an exact tie to the lower point for odd uppers — resolve
    # ties to the even index, as a hardware e2m1 conversion does
    mag = v.abs().clamp(max=6.0)
    idx = (mag.unsqueeze(-1) - grid).abs().argmin(-1)
    up = (idx + 1).clamp(max=7)
    tie = ((grid[up] - mag) == (mag - grid[idx])) & (idx % 2 == 1)
    idx = torch.where(tie, up, idx)
    code = (idx | ((v < 0) & (idx > 0)).long() << 3).to(torch.uint8).reshape(*x.shape[:-1], K // 2, 2)
    packed = code[..., 0] | (code[..., 1] << 4)
    return packed, (e + 127).to(torch.uint8)


def mxfp4_dequantize(packed: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """packed [..., K/2] uint8, scales [..., K/32] uint8 → [..., K] ``dtype``."""
    K = packed.shape[-1] * 2
    vals = _pair_lut(packed.device)[packed.long()].reshape(*packed.shape[:-1], K)
    s = torch.exp2(scales.float() - 127.0).repeat_interleave(BLOCK, dim=-1)
    return (vals * s).to(dtype)
