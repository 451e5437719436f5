"""Expert-weight layout utilities and checkpoint-format detection.

Grouped experts exist in two layouts: *standard* (separate ``w1``/``w3`` of shape
``[E, H, D]``) and *gmm* (fused ``w13`` of shape ``[E, 2H, D]``, rows ``[w1 | w3]``).
Checkpoints always use the standard layout; the fused layout is a run-time
detail of the grouped-GEMM converter.  Fusing / splitting goes through host
memory so the device never holds both copies, and is DTensor-aware: when the
parameter is sharded on dim 1, each rank fuses its own ``[w1_shard | w3_shard]``
halves (interleaved sharding) so no communication is needed.

Parity: torchtitan_npu/tools/weight_utils.py:17-272.
"""

from __future__ import annotations

import gc
import os

import torch
from torch.distributed.tensor import DTensor, Shard

__all__ = [
    "detect_expert_format",
    "convert_expert_format",
    "fuse_experts",
    "split_fused_experts",
    "is_dcp_checkpoint",
    "detect_input_format_by_path",
]


def detect_expert_format(state_dict: dict) -> str:
    """'gmm' if fused expert weights are present, 'standard' for w1/w3, 'none' without experts."""
    for key in state_dict:
        if "experts." in key or key.endswith((".w1", ".w13")):
            if ".gate_up_proj." in key or ".w13." in key or key.endswith(".w13"):
                return "gmm"
            if ".gate_proj." in key or ".w1." in key or key.endswith(".w1"):
                return "standard"
    return "none"


def is_dcp_checkpoint(path: str) -> bool:
    if os.path.exists(os.path.join(path, ".metadata")):
        return True
    try:
        return any(f.endswith(".distcp") for f in os.listdir(path))
    except OSError:
        return False


def detect_input_format_by_path(path: str) -> str:
    return "dcp" if is_dcp_checkpoint(path) else "hf"


def _sharded_on(t, dim: int) -> bool:
    return isinstance(t, DTensor) and any(isinstance(p, Shard) and p.dim == dim for p in t.placements)


def _fuse_pair(w1, w3):
    if isinstance(w1, DTensor):
        if w1.device_mesh != w3.device_mesh or w1.placements != w3.placements:
            raise ValueError("w1 and w3 must share mesh and placements to be fused")
        mesh, placements = w1.device_mesh, w1.placements
        dev = w1.device
        l1, l3 = w1.to_local().cpu(), w3.to_local().cpu()
        local = torch.cat([l1, l3], dim=1).to(dev)
        shape = torch.Size((w1.shape[0], w1.shape[1] + w3.shape[1], *w1.shape[2:]))
        stride = torch.empty(shape, device="meta").stride()
        return DTensor.from_local(local, mesh, placements, run_check=False, shape=shape, stride=stride)
    dev = w1.device
    return torch.cat([w1.cpu(), w3.cpu()], dim=1).to(dev)


def _split_one(w13):
    if isinstance(w13, DTensor):
        mesh, placements = w13.device_mesh, w13.placements
        local = w13.to_local()
        h = local.shape[1] // 2
        half_shape = torch.Size((w13.shape[0], w13.shape[1] // 2, *w13.shape[2:]))
        stride = torch.empty(half_shape, device="meta").stride()
        mk = lambda t: DTensor.from_local(t.contiguous().clone(), mesh, placements, run_check=False,  # noqa: E731
                                          shape=half_shape, stride=stride)
        return mk(local[:, :h]), mk(local[:, h:])
    a, b = torch.chunk(w13, 2, dim=1)
    return a.clone(), b.clone()


def fuse_experts(state_dict: dict) -> dict:
    """standard → gmm, in place: ``X.w1`` + ``X.w3`` → ``X.w13``."""
    for key in sorted(k for k in state_dict if k.endswith(".w1")):
        base = key[: -len(".w1")]
        k3 = base + ".w3"
        if k3 not in state_dict:
            continue
        w1, w3 = state_dict.pop(key), state_dict.pop(k3)
        state_dict[base + ".w13"] = _fuse_pair(w1, w3)
        del w1, w3
    gc.collect()
    return state_dict


def split_fused_experts(state_dict: dict) -> dict:
    """gmm → standard, in place: ``X.w13`` → ``X.w1``, ``X.w3``."""
    for key in [k for k in state_dict if k.endswith(".w13")]:
        base = key[: -len(".w13")]
        w1, w3 = _split_one(state_dict.pop(key))
        state_dict[base + ".w1"], state_dict[base + ".w3"] = w1, w3
    gc.collect()
    return state_dict


def convert_expert_format(state_dict: dict, target_format: str) -> dict:
    current = detect_expert_format(state_dict)
    if target_format == "gmm" and current == "standard":
        return fuse_experts(state_dict)
    if target_format == "standard" and current == "gmm":
        return split_fused_experts(state_dict)
    return state_dict
