"""Pipeline parallelism for decoder LLMs: split by layer FQNs, build NCCL-p2p schedules.

A model on the meta device is deep-copied per local stage and every module the stage does
not own is removed (``tok_embeddings`` lives on the first stage, ``norm`` + ``output`` on the
last; the embedding and head count as ``first/last_stage_less_layers`` layers when balancing).
Each stage is then parallelised (TP / AC / FSDP) with the model's own `parallelize_fn`.
Send/recv between stages stays on NCCL point-to-point, which overlaps with compute.

With FSDP inside a stage, each microbatch backward reshards parameters and reduce-scatters
gradients right away (rather than keeping all-gathered weights and unreduced grads for the
whole schedule), trading extra collectives for a flat memory profile.

Parity: upstream `pipeline_llm` as used by the reference (schedules such as ``1F1B``,
torchtitan_npu/models/deepseek_v3/config_registry.py:130-131), the reshard+sync-per-microbatch
behaviour (patches/torch/pipelining.py:84-162) and `input_ids` forwarding for hash-routed
models (models/deepseek_v4/pipeline_parallel.py:10-35).
"""

from __future__ import annotations

import copy
import math

import torch
import torch.nn as nn
from torch.distributed.pipelining import PipelineStage
from torch.distributed.pipelining.schedules import (
    PipelineScheduleMulti,
    PipelineScheduleSingle,
    ScheduleZBVZeroBubble,
    get_schedule_class,
)

from titan_b200.utils.logging import logger

__all__ = ["pipeline_llm", "generate_llm_fqn_per_model_part", "stage_ids_this_rank", "build_pipeline_schedule"]


def generate_llm_fqn_per_model_part(num_stages: int, num_layers: int, input_weight: int = 1,
                                    output_weight: int = 1) -> list[list[str]]:
    """Balanced assignment of ``tok_embeddings | layers.i | norm, output`` to `num_stages` stages."""
    if num_stages < 1:
        raise ValueError("num_stages must be >= 1")
    if num_stages == 1:
        return [["tok_embeddings", *[f"layers.{i}" for i in range(num_layers)], "norm", "output"]]
    effective = num_layers + input_weight + output_weight
    if num_stages > effective:
        raise ValueError(f"{num_stages} stages cannot be filled by {effective} effective layers")
    per, extra = divmod(effective, num_stages)
    if per <= max(input_weight, output_weight) and num_stages > 2 and per < max(input_weight, output_weight):
        raise ValueError("a stage would hold less than the embedding/head weight; lower the pp degree")
    out, cur = [], 0
    for s in range(num_stages):
        budget = per + (1 if s < extra else 0)
        names: list[str] = []
        if s == 0:
            names.append("tok_embeddings")
            budget -= input_weight
        if s == num_stages - 1:
            budget -= output_weight
        for _ in range(max(budget, 0)):
            if cur < num_layers:
                names.append(f"layers.{cur}")
                cur += 1
        if s == num_stages - 1:
            while cur < num_layers:
                names.append(f"layers.{cur}")
                cur += 1
            names += ["norm", "output"]
        out.append(names)
    return out


def stage_ids_this_rank(pp_rank: int, pp_size: int, num_stages: int, style: str = "loop") -> tuple[int, ...]:
    """Stages owned by a pp rank: ``loop`` = round-robin (interleaved schedules), ``v`` = V-shape (ZBV)."""
    if num_stages % pp_size != 0:
        raise ValueError(f"num_stages {num_stages} must be a multiple of pp degree {pp_size}")
    per_rank = num_stages // pp_size
    if style == "loop":
        return tuple(pp_rank + s * pp_size for s in range(per_rank))
    if style == "v":
        if per_rank != 2:
            raise ValueError("v-style schedules need exactly two stages per rank")
        return (pp_rank, num_stages - 1 - pp_rank)
    raise ValueError(f"unknown style {style!r}")


def _prune_to(model: nn.Module, fqns: list[str]) -> nn.Module:
    keep_layers = {f.split(".", 1)[1] for f in fqns if f.startswith("layers.")}
    top = {f for f in fqns if "." not in f}
    for name, child in list(model.named_children()):
        if name == "layers":
            for lname in list(child._modules.keys()):
                if lname not in keep_layers:
                    del child._modules[lname]
        elif isinstance(child, nn.Module) and name not in top and name in (
            "tok_embeddings", "norm", "output", "mtp_layers", "mtp_norm", "hc_head"
        ):
            setattr(model, name, None)
    return model


def build_pipeline_schedule(trainer_config, stages: list[PipelineStage], loss_fn, *, pp_size: int):
    par = trainer_config.parallelism
    cls = get_schedule_class(par.pipeline_parallel_schedule)
    looped = issubclass(cls, PipelineScheduleMulti)
    mb_size = par.pipeline_parallel_microbatch_size
    lbs = trainer_config.training.local_batch_size
    if lbs % mb_size != 0:
        raise ValueError(f"local_batch_size {lbs} must be divisible by pipeline microbatch size {mb_size}")
    n_mb = lbs // mb_size
    if n_mb < len(stages) * pp_size:
        logger.warning("%d microbatches < %d pipeline stages: the pipeline will bubble", n_mb, len(stages) * pp_size)
    sched = cls(stages if looped else stages[0], n_microbatches=n_mb, loss_fn=loss_fn, scale_grads=False)
    return sched


def pipeline_llm(model: nn.Module, *, parallel_dims, trainer_config, device, model_config, parallelize_fn, loss_fn):
    """→ (schedule, model_parts, has_first_stage, has_last_stage)."""
    pp_mesh = parallel_dims.get_mesh("pp")
    pp_rank, pp_size = pp_mesh.get_local_rank(), pp_mesh.size()
    par = trainer_config.parallelism
    cls = get_schedule_class(par.pipeline_parallel_schedule)
    looped = issubclass(cls, PipelineScheduleMulti)
    n_layers = model_config.n_layers
    in_w, out_w = par.pipeline_parallel_first_stage_less_layers, par.pipeline_parallel_last_stage_less_layers
    if par.pipeline_parallel_layers_per_stage is not None:
        num_stages = math.ceil((n_layers + in_w + out_w) / par.pipeline_parallel_layers_per_stage)
        if num_stages % pp_size:
            raise ValueError(f"{num_stages} stages is not a multiple of pp degree {pp_size}")
    else:
        num_stages = pp_size * (2 if looped else 1)
    if not looped and num_stages != pp_size:
        raise ValueError(f"schedule {cls.__name__} runs one stage per rank; got {num_stages} stages")
    fqns = generate_llm_fqn_per_model_part(num_stages, n_layers, in_w, out_w)
    style = "v" if cls is ScheduleZBVZeroBubble else "loop"
    stages, parts = [], []
    for sid in stage_ids_this_rank(pp_rank, pp_size, num_stages, style):
        part = _prune_to(copy.deepcopy(model), fqns[sid])
        part = parallelize_fn(part, parallel_dims=parallel_dims, training=trainer_config.training,
                              model_converters=trainer_config.model_converters, parallelism=par,
                              compile_config=trainer_config.compile, ac_config=trainer_config.activation_checkpoint,
                              dump_folder=trainer_config.job.dump_folder)
        stages.append(PipelineStage(part, sid, num_stages, device, group=pp_mesh.get_group()))
        parts.append(part)
        logger.info("pp rank %d builds stage %d with %s", pp_rank, sid, fqns[sid])
    schedule = build_pipeline_schedule(trainer_config, stages, loss_fn, pp_size=pp_size)
    has_first = any(s.is_first for s in stages)
    has_last = any(s.is_last for s in stages)
    _force_reshard_per_microbatch(parts)
    for stage in stages:
        _sync_every_microbatch(stage)
    return schedule, parts, has_first, has_last


def _force_reshard_per_microbatch(parts: list[nn.Module]) -> None:
    """Make FSDP reshard and reduce-scatter after every microbatch backward of a stage."""
    from torch.distributed.fsdp import FSDPModule

    for part in parts:
        for m in part.modules():
            if isinstance(m, FSDPModule):
                m.set_reshard_after_backward(True)
                m.set_requires_gradient_sync(True)
                m.set_is_last_backward(True)


def _sync_every_microbatch(stage: PipelineStage) -> None:
    """Replace the stage's `backward_maybe_with_nosync`: the stock version switches FSDP's reshard / gradient sync OFF
    for every microbatch and reduces once at the end of the step, which keeps a stage's unsharded parameters and
    full-size gradients alive across all microbatches.  Here every microbatch backward reduce-scatters into the
    sharded gradient and reshards the parameters (parity: torchtitan_npu/patches/torch/pipelining.py:100-162,
    "always reshard + sync")."""
    from torch.distributed.fsdp import FSDPModule
    from torch.distributed.pipelining._backward import stage_backward, stage_backward_input, stage_backward_weight

    stock = stage.backward_maybe_with_nosync

    def backward(backward_type, bwd_kwargs: dict, last_backward: bool = False):
        sub = stage.submod
        if not isinstance(sub, FSDPModule):
            return stock(backward_type, bwd_kwargs, last_backward=last_backward)
        sub.set_is_last_backward(True)
        sub.set_reshard_after_backward(True)
        sub.set_requires_gradient_sync(True)
        if backward_type == "full":
            return stage_backward(bwd_kwargs["stage_output"], bwd_kwargs["output_grads"],
                                  bwd_kwargs["input_values"]), None
        if backward_type == "input":
            return stage_backward_input(bwd_kwargs["stage_output"], bwd_kwargs["output_grads"],
                                        bwd_kwargs["input_values"], sub.parameters())
        if backward_type == "weight":
            return stage_backward_weight(sub.parameters(), bwd_kwargs["param_groups"]), None
        raise RuntimeError(f"unknown backward type {backward_type!r}")

    stage.backward_maybe_with_nosync = backward
