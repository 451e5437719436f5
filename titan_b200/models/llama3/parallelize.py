"""Parallelisation of Llama-3: TP(+SP, loss parallel) → AC → compile → FSDP2/HSDP or replicate.

Parity: the upstream-equivalent `parallelize_fn(model, *, parallel_dims, training,
model_converters, parallelism, compile_config, ac_config, dump_folder)` contract
the reference's recipes rely on (torchtitan_npu/models/deepseek_v32/parallelize.py:127-137).
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch.distributed.tensor import Replicate, Shard
from torch.distributed.tensor.parallel import (
    ColwiseParallel,
    PrepareModuleInput,
    RowwiseParallel,
    SequenceParallel,
)

from titan_b200.parallel.activation_checkpoint import apply_ac
from titan_b200.parallel.fsdp import DTYPE_MAP, apply_fsdp, apply_replicate
from titan_b200.parallel.tensor_parallel import maybe_enable_async_tp, parallelize_module

__all__ = ["parallelize_llama", "apply_tp", "apply_compile"]


def apply_tp(model: nn.Module, tp_mesh, *, loss_parallel: bool, async_tp: bool = False) -> None:
    parallelize_module(
        model,
        tp_mesh,
        {
            "tok_embeddings": RowwiseParallel(input_layouts=Replicate(), output_layouts=Shard(1)),
            "norm": SequenceParallel(),
            "output": ColwiseParallel(
                input_layouts=Shard(1),
                output_layouts=Shard(-1) if loss_parallel else Replicate(),
                use_local_output=not loss_parallel,
            ),
        },
    )
    if async_tp:
        # fused sequence-parallel linears: weights keep the column / row shards, but no module-level gather or
        # scatter hooks; the sub-layers exchange plain sequence-sharded tensors and the collectives run inside the
        # all-gather→GEMM / GEMM→reduce-scatter kernels
        from titan_b200.parallel.async_tp import enable_for_llama
        from titan_b200.parallel.tensor_parallel import ShardOnly

        for block in model.layers.values():
            parallelize_module(block, tp_mesh, {
                "attention_norm": SequenceParallel(use_local_output=True),
                "attention.wq": ShardOnly(0), "attention.wk": ShardOnly(0), "attention.wv": ShardOnly(0),
                "attention.wo": ShardOnly(1),
                "ffn_norm": SequenceParallel(use_local_output=True),
                "feed_forward.w1": ShardOnly(0), "feed_forward.w3": ShardOnly(0), "feed_forward.w2": ShardOnly(1),
            })
        enable_for_llama(model, tp_mesh)
        return
    for block in model.layers.values():
        plan = {
            "attention_norm": SequenceParallel(),
            "attention": PrepareModuleInput(
                input_layouts=(Shard(1), None, None, None),
                desired_input_layouts=(Replicate(), None, None, None),
            ),
            "attention.wq": ColwiseParallel(),
            "attention.wk": ColwiseParallel(),
            "attention.wv": ColwiseParallel(),
            "attention.wo": RowwiseParallel(output_layouts=Shard(1)),
            "ffn_norm": SequenceParallel(),
            "feed_forward": PrepareModuleInput(input_layouts=(Shard(1),), desired_input_layouts=(Replicate(),)),
            "feed_forward.w1": ColwiseParallel(),
            "feed_forward.w2": RowwiseParallel(output_layouts=Shard(1)),
            "feed_forward.w3": ColwiseParallel(),
        }
        parallelize_module(block, tp_mesh, plan)


def apply_compile(model: nn.Module, compile_config) -> None:
    for name, block in list(model.layers.named_children()):
        model.layers.register_module(name, torch.compile(block, backend=compile_config.backend, fullgraph=True))


def parallelize_llama(
    model: nn.Module,
    *,
    parallel_dims,
    training,
    model_converters=None,
    parallelism=None,
    compile_config=None,
    ac_config=None,
    dump_folder: str = "",
):
    if training.seq_len % parallel_dims.seq_len_divisor != 0:
        raise ValueError(
            f"seq_len {training.seq_len} must be divisible by tp * 2 * cp = {parallel_dims.seq_len_divisor}"
        )
    if parallel_dims.tp_enabled:
        tp_mesh = parallel_dims.get_mesh("tp")
        async_tp = maybe_enable_async_tp(parallelism, tp_mesh)
        apply_tp(model, tp_mesh, loss_parallel=not parallelism.disable_loss_parallel, async_tp=async_tp)

    if ac_config is not None and ac_config.mode != "none":
        apply_ac(model, ac_config)

    if compile_config is not None and compile_config.enable and "model" in compile_config.components:
        apply_compile(model, compile_config)

    if parallel_dims.fsdp_enabled:
        names = ("dp_replicate", "fsdp") if parallel_dims.dp_replicate_enabled else None
        dp_mesh = parallel_dims.get_mesh(names) if names else parallel_dims.get_mesh("fsdp")
        ignored = None
        if getattr(parallelism, "fsdp_fused_collectives", False):
            if parallel_dims.tp_enabled or parallel_dims.dp_replicate_enabled:
                raise NotImplementedError("fsdp_fused_collectives composes with plain FSDP only (no TP / HSDP)")
            from titan_b200.parallel.fused_fsdp import shard_linears

            ignored = set(shard_linears(model, dp_mesh))
        apply_fsdp(
            model,
            dp_mesh,
            ignored_params=ignored,
            param_dtype=DTYPE_MAP[training.mixed_precision_param],
            reduce_dtype=DTYPE_MAP[training.mixed_precision_reduce],
            pp_enabled=parallel_dims.pp_enabled,
            cpu_offload=training.enable_cpu_offload,
            reshard_after_forward_policy=parallelism.fsdp_reshard_after_forward,
        )
    elif parallel_dims.dp_replicate_enabled:
        apply_replicate(
            model,
            parallel_dims.get_mesh("dp_replicate"),
            param_dtype=DTYPE_MAP[training.mixed_precision_param],
            reduce_dtype=DTYPE_MAP[training.mixed_precision_reduce],
        )
    return model
