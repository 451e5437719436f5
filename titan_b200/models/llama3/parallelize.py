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


def apply_ulysses_cp(model: nn.Module, parallel_dims, parallelism, *, rope: str) -> None:
    """Ulysses context parallelism on every block's attention: hooks around the attention core, or (with
    ``parallelism.context_parallel_fused_projections``) the exchanges folded into the projections."""
    from titan_b200.parallel.context_parallel import apply_cp_to_attention_module

    cp_mesh = parallel_dims.get_mesh("cp")
    blocks = [b for b in model.layers.values() if b is not None]
    for b in blocks:
        a = b.attention
        tp = parallel_dims.tp if parallel_dims.tp_enabled else 1
        for what, n in (("n_heads", a.n_heads), ("n_kv_heads", a.n_kv_heads)):
            if (n // tp) % parallel_dims.cp != 0:
                raise ValueError(f"[Ulysses CP] {what}={n} (per TP rank {n // tp}) must be divisible by "
                                 f"context_parallel_degree={parallel_dims.cp}.")
    if getattr(parallelism, "context_parallel_fused_projections", False):
        if parallel_dims.tp_enabled:
            raise NotImplementedError("context_parallel_fused_projections does not compose with tensor parallelism")
        from titan_b200.models.common.rope import apply_rotary_emb_complex, apply_rotary_emb_cos_sin
        from titan_b200.parallel.context_parallel.ulysses import apply_fused_ulysses

        rope_fn = apply_rotary_emb_complex if rope == "complex" else apply_rotary_emb_cos_sin
        for b in blocks:
            apply_fused_ulysses(b.attention, cp_mesh, rope_fn)
    else:
        apply_cp_to_attention_module([b.attention.inner_attention for b in blocks], cp_mesh)


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

    if parallel_dims.cp_enabled:
        apply_ulysses_cp(model, parallel_dims, parallelism, rope="complex")

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
            reduce_scatter=parallelism.fsdp_reduce_scatter,
            all_gather=parallelism.fsdp_all_gather,
        )
    elif parallel_dims.dp_replicate_enabled:
        apply_replicate(
            model,
            parallel_dims.get_mesh(("dp_replicate", "fsdp")),
            param_dtype=DTYPE_MAP[training.mixed_precision_param],
            reduce_dtype=DTYPE_MAP[training.mixed_precision_reduce],
        )
    return model
