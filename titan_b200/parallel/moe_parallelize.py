"""Shared MoE parallelisation: tensor-parallel plan for the MoE block (tokens stay sequence-sharded
around the block) and the expert plan chosen from (tp, ep, etp) and the configured comm backend.

Parity: torchtitan_npu/models/common/moe_parallelize.py:31-120
(`apply_sequence_sharded_moe_ep_tp`; DeepEP / HybridEP / TorchAO pass-throughs become the
`fused_p2p` backend here; unknown backends raise).
"""

from __future__ import annotations

import torch.nn as nn
from torch.distributed.tensor import Partial, Replicate, Shard
from torch.distributed.tensor.parallel import PrepareModuleInputOutput

from titan_b200.parallel.expert_parallel import (
    ExpertParallel,
    ExpertTensorParallel,
    FusedExpertParallel,
    TensorParallel,
)
from titan_b200.parallel.tensor_parallel import NoParallel, parallelize_module

__all__ = ["apply_moe_ep_tp", "expert_style_for"]


def expert_style_for(*, tp: bool, ep: bool, etp: bool, comm_backend: str = "standard"):
    if comm_backend in ("deepep", "hybridep", "torchao"):
        raise NotImplementedError(
            f"expert_parallel_comm_backend={comm_backend!r} is a third-party library path that this framework does "
            "not ship; use 'standard' (NCCL all-to-all) or 'fused_p2p' (in-kernel peer-memory dispatch)")
    if ep and etp:
        return ExpertTensorParallel()
    if ep:
        return FusedExpertParallel() if comm_backend == "fused_p2p" else ExpertParallel()
    if tp:
        return TensorParallel()
    return None


def apply_moe_ep_tp(model: nn.Module, *, tp_mesh=None, ep_mesh=None, etp_mesh=None, ep_etp_mesh=None,
                    comm_backend: str = "standard", layers_attr: str = "layers", extra_moe_inputs: int = 0) -> None:
    """``extra_moe_inputs``: positional inputs after the tokens that pass through untouched (DeepSeek-V4 hands the
    token ids to the MoE block for hash routing)."""
    none = (None,) * extra_moe_inputs
    if ep_mesh is not None and comm_backend == "fused_p2p":
        from titan_b200.ops import moe_comm
        from titan_b200.trainer import stash

        cfg = stash.get_trainer_config()
        if cfg is not None:
            moe_comm.set_capacity_factor(cfg.parallelism.expert_parallel_capacity_factor)
    for block in getattr(model, layers_attr).values():
        if block is None or not getattr(block, "moe_enabled", False):
            continue
        moe = block.moe
        if tp_mesh is not None:
            plan = {
                # tokens enter sequence-sharded, are gathered for routing, and leave as partial sums that are
                # reduce-scattered back to the sequence shard
                "moe": PrepareModuleInputOutput(
                    input_layouts=(Shard(1), *none), desired_input_layouts=(Replicate(), *none), use_local_input=True,
                    output_layouts=(Partial(),), desired_output_layouts=(Shard(1),)),
                "moe.router.gate": NoParallel(),
            }
            if moe.shared_experts is not None:
                from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel

                plan.update({"moe.shared_experts.w1": ColwiseParallel(),
                             "moe.shared_experts.w2": RowwiseParallel(output_layouts=Partial()),
                             "moe.shared_experts.w3": ColwiseParallel()})
            parallelize_module(block, tp_mesh, plan)
        style = expert_style_for(tp=tp_mesh is not None and etp_mesh is not None, ep=ep_mesh is not None,
                                 etp=etp_mesh is not None and ep_mesh is not None, comm_backend=comm_backend)
        if style is None:
            continue
        if isinstance(style, ExpertTensorParallel):
            mesh = ep_etp_mesh
        elif isinstance(style, ExpertParallel):
            mesh = ep_mesh
        else:
            mesh = tp_mesh
        parallelize_module(moe.experts, mesh, style)
