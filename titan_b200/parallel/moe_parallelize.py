"""Shared MoE parallelisation: tensor-parallel plan for the MoE block (tokens stay sequence-sharded
around the block) and the expert plan chosen from (tp, ep, etp) and the configured comm backend.

Parity: torchtitan_npu/models/common/moe_parallelize.py:31-120
(`apply_sequence_sharded_moe_ep_tp`; DeepEP / HybridEP / TorchAO pass-throughs become the
`fused_p2p` backend here; unknown backends raise).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.tensor import Partial, Replicate, Shard
from torch.distributed.tensor.parallel import PrepareModuleInputOutput

from titan_b200.parallel.expert_parallel import (
    ExpertParallel,
    ExpertTensorParallel,
    FusedExpertParallel,
    TensorParallel,
)
from titan_b200.parallel.tensor_parallel import NoParallel, ReplicateParams, parallelize_module

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


def _slice_to_local_sequence(group, world: int):
    """Pre-hook for the sequence-sharded form: extra inputs that carry the FULL sequence (token ids for hash routing)
    are cut to this rank's slice so that they line up with the local tokens."""
    rank = dist.get_rank(group)

    def hook(mod, args):
        x = args[0]
        out = [x]
        for extra in args[1:]:
            if isinstance(extra, torch.Tensor) and extra.dim() >= 2 and extra.shape[1] == x.shape[1] * world:
                extra = extra.chunk(world, dim=1)[rank]
            out.append(extra)
        return tuple(out)

    return hook


def apply_moe_ep_tp(model: nn.Module, *, tp_mesh=None, ep_mesh=None, etp_mesh=None, ep_etp_mesh=None,
                    comm_backend: str = "standard", layers_attr: str = "layers", extra_moe_inputs: int = 0) -> None:
    """Two token layouts under tensor parallelism:

    * experts split over tp (no EP) or over etp (EP x ETP): the tokens are all-gathered at the block boundary, every
      rank routes all of them through its hidden slice of the experts, and the block output (routed + shared) is a
      partial sum that the reduce-scatter back to the sequence shard adds up;
    * EP that borrows the tp ranks (etp = 1): the tokens stay sequence-sharded through the block (each rank routes
      and dispatches its own slice only), the router weight sees per-rank tokens (gradient summed over tp), and the
      shared experts gather their own input and reduce-scatter their own output.

    ``extra_moe_inputs``: positional inputs after the tokens that pass through untouched (DeepSeek-V4 hands the
    token ids to the MoE block for hash routing)."""
    none = (None,) * extra_moe_inputs
    if ep_mesh is not None and comm_backend == "fused_p2p":
        from titan_b200.ops import moe_comm
        from titan_b200.trainer import stash

        cfg = stash.get_trainer_config()
        if cfg is not None:
            moe_comm.set_capacity_factor(cfg.parallelism.expert_parallel_capacity_factor)
    etp_on = ep_mesh is not None and etp_mesh is not None and etp_mesh.size() > 1
    seq_sharded = tp_mesh is not None and ep_mesh is not None and not etp_on
    for block in getattr(model, layers_attr).values():
        if block is None or not getattr(block, "moe_enabled", False):
            continue
        moe = block.moe
        if tp_mesh is not None:
            from torch.distributed.tensor.parallel import ColwiseParallel, PrepareModuleInput, RowwiseParallel

            if seq_sharded:
                plan = {
                    "moe": PrepareModuleInputOutput(
                        input_layouts=(Shard(1), *none), desired_input_layouts=(Shard(1), *none), use_local_input=True,
                        output_layouts=(Shard(1),), desired_output_layouts=(Shard(1),)),
                    "moe.router.gate": ReplicateParams(),
                }
                if moe.shared_experts is not None:
                    plan.update({
                        "moe.shared_experts": PrepareModuleInput(input_layouts=(Shard(0),),
                                                                 desired_input_layouts=(Replicate(),)),
                        "moe.shared_experts.w1": ColwiseParallel(),
                        "moe.shared_experts.w2": RowwiseParallel(output_layouts=Shard(0)),
                        "moe.shared_experts.w3": ColwiseParallel()})
                moe.router.tokens_sharded = True
                moe.counts_group = tp_mesh.get_group()   # per-expert token counts are per-rank slices
                if extra_moe_inputs:
                    moe.register_forward_pre_hook(_slice_to_local_sequence(tp_mesh.get_group(), tp_mesh.size()))
            else:
                plan = {
                    "moe": PrepareModuleInputOutput(
                        input_layouts=(Shard(1), *none), desired_input_layouts=(Replicate(), *none),
                        use_local_input=True, output_layouts=(Partial(),), desired_output_layouts=(Shard(1),)),
                    "moe.router.gate": NoParallel(),
                }
                if moe.shared_experts is not None:
                    plan.update({"moe.shared_experts.w1": ColwiseParallel(),
                                 "moe.shared_experts.w2": RowwiseParallel(output_layouts=Partial()),
                                 "moe.shared_experts.w3": ColwiseParallel()})
                # routed outputs are partial sums over tp: gate values applied AFTER the experts get partial gradients
                moe.tp_partial_group = tp_mesh.get_group()
            parallelize_module(block, tp_mesh, plan)
        style = expert_style_for(tp=tp_mesh is not None and ep_mesh is None, ep=ep_mesh is not None, etp=etp_on,
                                 comm_backend=comm_backend)
        if style is None:
            continue
        if isinstance(style, ExpertTensorParallel):
            mesh = ep_etp_mesh
        elif isinstance(style, ExpertParallel):
            mesh = ep_mesh
        else:
            mesh = tp_mesh
        parallelize_module(moe.experts, mesh, style)
