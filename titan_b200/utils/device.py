"""Device identification and peak-throughput table used for MFU.

Parity: torchtitan_npu/tools/device.py:8-32 (device-name → generation) and the peak
FLOPS table keyed by device name (patches/tools/metrics.py:42-53).
"""

from __future__ import annotations

import json
import os

import torch

__all__ = ["device_generation", "get_peak_flops", "PEAK_DENSE_FLOPS", "measured_peaks", "HBM_BYTES"]

# dense (no 2:4 sparsity) tensor-core peaks per GPU
PEAK_DENSE_FLOPS = {
    "B200": {"bf16": 2.25e15, "fp8": 4.5e15, "fp4": 9.0e15, "tf32": 1.1e15},
    "H100": {"bf16": 989e12, "fp8": 1979e12, "tf32": 494e12},
    "H200": {"bf16": 989e12, "fp8": 1979e12, "tf32": 494e12},
    "A100": {"bf16": 312e12, "tf32": 156e12},
}
HBM_BYTES = {"B200": 180 * 10**9, "H100": 80 * 10**9, "H200": 141 * 10**9, "A100": 80 * 10**9}


def device_generation(name: str | None = None) -> str:
    if name is None:
        name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    up = name.upper()
    for key in ("B200", "H200", "H100", "A100"):
        if key in up:
            return key
    return "unknown"


def measured_peaks(path: str | None = None) -> dict | None:
    """Measured copy bandwidth / cuBLAS throughput of this machine, if a record exists beside the repo root."""
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = path or os.path.join(here, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return None


def get_peak_flops(name: str | None = None, dtype: str = "bf16") -> float:
    gen = device_generation(name)
    table = PEAK_DENSE_FLOPS.get(gen)
    if table is None:
        return PEAK_DENSE_FLOPS["B200"][dtype] if gen == "unknown" and torch.cuda.is_available() else 1e12
    return table.get(dtype, table["bf16"])
