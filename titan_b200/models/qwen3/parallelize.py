"""Parallelisation of Qwen3: TP/SP, Ulysses context parallelism on the attention core, EP for MoE flavors, AC, FSDP2.

Parity: torchtitan_npu/models/qwen3/parallelize.py:22-63 (the head-divisibility checks of Ulysses CP and the swap
of the upstream ring-attention CP for the registry strategy) on top of the upstream Qwen3 plan.
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
from titan_b200.parallel.moe_parallelize import apply_moe_ep_tp
from titan_b200.parallel.tensor_parallel import ReplicateParams, maybe_enable_async_tp, parallelize_module
from titan_b200.utils.logging import logger

__all__ = ["parallelize_qwen3", "apply_non_moe_tp", "validate_ulysses"]


def validate_ulysses(model, cp_degree: int) -> None:
    first = next(iter(model.layers.values()))
    n_heads, n_kv = first.attention.n_heads, first.attention.n_kv_heads
    if n_heads % cp_degree != 0:
        raise ValueError(f"[Ulysses CP] n_heads={n_heads} must be divisible by context_parallel_degree={cp_degree}.")
    if n_kv % cp_degree != 0:
        raise ValueError(f"[Ulysses CP] n_kv_heads={n_kv} must be divisible by context_parallel_degree={cp_degree}.")
    logger.info("[Ulysses CP] Qwen3 Ulysses CP enabled: cp_degree=%d, n_heads=%d", cp_degree, n_heads)


def apply_non_moe_tp(model: nn.Module, tp_mesh, *, loss_parallel: bool) -> None:
    if model.config.enable_weight_tying:
        raise NotImplementedError("tensor parallelism with tied embeddings is not supported: the embedding is "
                                  "row-sharded and the output projection column-sharded")
    parallelize_module(model, tp_mesh, {
        "tok_embeddings": RowwiseParallel(input_layouts=Replicate(), output_layouts=Shard(1)),
        "norm": SequenceParallel(),
        "output": ColwiseParallel(input_layouts=Shard(1), output_layouts=Shard(-1) if loss_parallel else Replicate(),
                                  use_local_output=not loss_parallel),
    })
    for block in model.layers.values():
        plan = {
            "attention_norm": SequenceParallel(),
            "attention": PrepareModuleInput(input_layouts=(Shard(1), None, None, None),
                                            desired_input_layouts=(Replicate(), None, None, None)),
            "attention.wq": ColwiseParallel(),
            "attention.wk": ColwiseParallel(),
            "attention.wv": ColwiseParallel(),
            # per-head norms act on the head dim of local heads: weights replicated, activations head-sharded
            "attention.q_norm": ReplicateParams(),
            "attention.k_norm": ReplicateParams(),
            "attention.wo": RowwiseParallel(output_layouts=Shard(1)),
            "ffn_norm": SequenceParallel(),
        }
        if block.attention.q_norm is None:
            plan.pop("attention.q_norm"), plan.pop("attention.k_norm")
        if not block.moe_enabled:
            plan.update({
                "feed_forward": PrepareModuleInput(input_layouts=(Shard(1),), desired_input_layouts=(Replicate(),)),
                "feed_forward.w1": ColwiseParallel(),
                "feed_forward.w2": RowwiseParallel(output_layouts=Shard(1)),
                "feed_forward.w3": ColwiseParallel(),
            })
        parallelize_module(block, tp_mesh, plan)


def parallelize_qwen3(model: nn.Module, *, parallel_dims, training, model_converters=None, parallelism=None,
                      compile_config=None, ac_config=None, dump_folder: str = ""):
    pd = parallel_dims
    if training.seq_len % pd.seq_len_divisor != 0:
        raise ValueError(f"seq_len {training.seq_len} must be divisible by tp * 2 * cp = {pd.seq_len_divisor}")
    tp_mesh = pd.get_optional_mesh("tp")
    if tp_mesh is not None:
        maybe_enable_async_tp(parallelism, tp_mesh)
        apply_non_moe_tp(model, tp_mesh, loss_parallel=not parallelism.disable_loss_parallel)
    if pd.cp_enabled:
        from titan_b200.parallel.context_parallel import apply_cp_to_attention_module

        validate_ulysses(model, pd.cp)
        if getattr(parallelism, "context_parallel_fused_projections", False):
            if tp_mesh is not None:
                raise NotImplementedError("context_parallel_fused_projections does not compose with tensor "
                                          "parallelism")
            from titan_b200.models.common.rope import apply_rotary_emb_cos_sin
            from titan_b200.parallel.context_parallel.ulysses import apply_fused_ulysses

            for b in model.layers.values():
                apply_fused_ulysses(b.attention, pd.get_mesh("cp"), apply_rotary_emb_cos_sin)
        else:
            apply_cp_to_attention_module([b.attention.inner_attention for b in model.layers.values()],
                                         pd.get_mesh("cp"))
    if model.config.moe_enabled and (tp_mesh is not None or pd.ep_enabled):
        ep_etp = pd._sparse["ep", "etp"] if (pd.ep_enabled and pd.etp_enabled) else None
        apply_moe_ep_tp(model, tp_mesh=tp_mesh, ep_mesh=pd.get_optional_mesh("ep"),
                        etp_mesh=pd.get_optional_mesh("etp") if pd.etp_enabled else None, ep_etp_mesh=ep_etp,
                        comm_backend=parallelism.expert_parallel_comm_backend)
    if ac_config is not None and ac_config.mode != "none":
        apply_ac(model, ac_config)
    if compile_config is not None and compile_config.enable and "model" in compile_config.components:
        for name, block in list(model.layers.named_children()):
            if not block.moe_enabled:
                model.layers.register_module(name, torch.compile(block, backend=compile_config.backend))
    if pd.fsdp_enabled or pd.ep_enabled:
        names = ("dp_replicate", "fsdp") if pd.dp_replicate_enabled else None
        dp_mesh = pd.get_mesh(names) if names else pd.get_optional_mesh("fsdp")
        if dp_mesh is not None:
            edp = pd.mesh_even_if_trivial("efsdp") if pd.ep_enabled else None
            apply_fsdp(model, dp_mesh, param_dtype=DTYPE_MAP[training.mixed_precision_param],
                       reduce_dtype=DTYPE_MAP[training.mixed_precision_reduce], pp_enabled=pd.pp_enabled,
                       cpu_offload=training.enable_cpu_offload,
                       reshard_after_forward_policy=parallelism.fsdp_reshard_after_forward,
            reduce_scatter=parallelism.fsdp_reduce_scatter,
            all_gather=parallelism.fsdp_all_gather,
                       ep_degree=pd.ep if edp is not None else 1, edp_mesh=edp,
                       gradient_divide_factor=pd.fsdp_gradient_divide_factor)
    elif pd.dp_replicate_enabled:
        apply_replicate(model, pd.get_mesh(("dp_replicate", "fsdp")), param_dtype=DTYPE_MAP[training.mixed_precision_param],
                        reduce_dtype=DTYPE_MAP[training.mixed_precision_reduce])
    return model
