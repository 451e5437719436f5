"""Parallelisation of DeepSeek-V3.2: TP/SP plan for the three-stage attention, DSA context parallelism,
EP for experts, AC, FSDP2, and the distributed indexer-loss tracker.

TP plan: ``wq_b`` / ``wkv_b`` column-parallel (heads split), ``wo`` row-parallel; the latent projections
(``wq_a, q_norm, wkv_a, kv_norm``) and the whole indexer stay replicated (`NoParallel`): they produce per-token
latents shared by all heads.  The attention core receives head-split queries and the replicated one-head KV
latent; its K/V gradients are partial sums over TP ranks and are all-reduced in backward
(`PrepareModuleInputOutputWithBwdAllReduce`).

Parity: torchtitan_npu/models/deepseek_v32/parallelize.py:57-630 (asserts :141-154, TP plan :299-514,
CP :195-212, indexer-loss tracking :517-565).
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

from titan_b200.models.common.dsa_indexer_loss import DSAIndexerLossAutoScaler, DSAIndexerLossLoggingHelper
from titan_b200.parallel.activation_checkpoint import apply_ac
from titan_b200.parallel.fsdp import DTYPE_MAP, apply_fsdp, apply_replicate
from titan_b200.parallel.moe_parallelize import apply_moe_ep_tp
from titan_b200.parallel.tensor_parallel import (
    AwaitRowwiseParallel,
    NoParallel,
    PrepareModuleInputOutputWithBwdAllReduce,
    maybe_enable_async_tp,
    parallelize_module,
)
from titan_b200.protocols.converter import has_converter
from titan_b200.trainer import stash

__all__ = ["parallelize_deepseekv32", "apply_non_moe_tp", "apply_distributed_indexer_loss_tracking"]


def _blocks(model):
    out = list(model.layers.values())
    out += [m.block for m in getattr(model, "mtp_layers", {}).values()]
    return [b for b in out if b is not None]


def apply_non_moe_tp(model: nn.Module, tp_mesh, *, loss_parallel: bool) -> None:
    parallelize_module(model, tp_mesh, {
        "tok_embeddings": RowwiseParallel(input_layouts=Replicate(), output_layouts=Shard(1)),
        "norm": SequenceParallel(),
        "output": ColwiseParallel(input_layouts=Shard(1), output_layouts=Shard(-1) if loss_parallel else Replicate(),
                                  use_local_output=not loss_parallel),
    })
    for block in _blocks(model):
        plan = {
            "attention_norm": SequenceParallel(),
            "attention": PrepareModuleInput(input_layouts=(Shard(1), None, None, None, None),
                                            desired_input_layouts=(Replicate(), None, None, None, None)),
            "attention.pre_attention.wq_a": NoParallel(),
            "attention.pre_attention.q_norm": NoParallel(),
            "attention.pre_attention.wq_b": ColwiseParallel(),
            "attention.pre_attention.wkv_a": NoParallel(),
            "attention.pre_attention.kv_norm": NoParallel(),
            "attention.pre_attention.wkv_b": ColwiseParallel(),
            "attention.pre_attention.indexer.wq_b": NoParallel(),
            "attention.pre_attention.indexer.wk": NoParallel(),
            "attention.pre_attention.indexer.k_norm": NoParallel(),
            "attention.pre_attention.indexer.weights_proj": NoParallel(),
            # k (arg 1) and v (arg 2) are replicated latents read by every rank's heads
            "attention.inner_attention": PrepareModuleInputOutputWithBwdAllReduce(
                bwd_allreduce_input_idx=(1, 2), input_layouts=None, desired_input_layouts=None,
                output_layouts=None, desired_output_layouts=None),
            "attention.post_attention.wo": AwaitRowwiseParallel(output_layouts=Shard(1)),
            "ffn_norm": SequenceParallel(),
        }
        if not block.moe_enabled:
            plan.update({
                "feed_forward": PrepareModuleInput(input_layouts=(Shard(1),), desired_input_layouts=(Replicate(),)),
                "feed_forward.w1": ColwiseParallel(),
                "feed_forward.w2": RowwiseParallel(output_layouts=Shard(1)),
                "feed_forward.w3": ColwiseParallel(),
            })
        parallelize_module(block, tp_mesh, plan)


def apply_distributed_indexer_loss_tracking(parallel_dims) -> None:
    """Log the mean indexer loss on log steps with ONE all-reduce of the per-layer vector."""
    import torch.distributed as dist

    def hook(trainer):
        loss_mesh = parallel_dims.get_optional_mesh("loss") if dist.is_initialized() else None
        pp_mesh = parallel_dims.get_optional_mesh("pp") if dist.is_initialized() else None
        v = DSAIndexerLossLoggingHelper.reduce_and_pop(trainer.gradient_accumulation_steps, loss_mesh, pp_mesh)
        return {} if v is None else {"loss_metrics/indexer_loss": v}

    stash.register_metrics_hook(hook)


def parallelize_deepseekv32(model: nn.Module, *, parallel_dims, training, model_converters=None, parallelism=None,
                            compile_config=None, ac_config=None, dump_folder: str = ""):
    pd = parallel_dims
    if training.seq_len % pd.seq_len_divisor != 0:
        raise ValueError(f"seq_len {training.seq_len} must be divisible by tp * 2 * cp = {pd.seq_len_divisor}")
    convs = model_converters.converters if model_converters is not None else []
    if pd.tp_enabled and not pd.ep_enabled and has_converter(convs, "b200_gmm"):
        raise ValueError("the grouped-GEMM converter needs expert parallelism when tensor parallelism is on")
    # the indexer KL term must not be counted once per accumulation step and rank
    grad_accum = max(training.global_batch_size // max(training.local_batch_size * pd.dp_degree, 1), 1) \
        if training.global_batch_size > 0 else 1
    DSAIndexerLossAutoScaler.set_loss_scale(1.0 / (grad_accum * pd.dp_replicate * pd.dp_shard * pd.cp))
    apply_distributed_indexer_loss_tracking(pd)

    tp_mesh = pd.get_optional_mesh("tp")
    if tp_mesh is not None:
        maybe_enable_async_tp(parallelism, tp_mesh)
        apply_non_moe_tp(model, tp_mesh, loss_parallel=not parallelism.disable_loss_parallel)
    if pd.cp_enabled:
        from titan_b200.parallel.context_parallel import apply_cp_to_attention_module
        from titan_b200.parallel.context_parallel import sparse_attention_cp  # noqa: F401  (registers the strategy)

        apply_cp_to_attention_module([b.attention.inner_attention for b in _blocks(model)], pd.get_mesh("cp"))
    if tp_mesh is not None or pd.ep_enabled:
        ep_etp = pd._sparse["ep", "etp"] if (pd.ep_enabled and pd.etp_enabled) else None
        apply_moe_ep_tp(model, tp_mesh=tp_mesh, ep_mesh=pd.get_optional_mesh("ep"),
                        etp_mesh=pd.get_optional_mesh("etp") if pd.etp_enabled else None, ep_etp_mesh=ep_etp,
                        comm_backend=parallelism.expert_parallel_comm_backend)
    if ac_config is not None and ac_config.mode != "none":
        apply_ac(model, ac_config)
        if len(getattr(model, "mtp_layers", {})):
            apply_ac(model, ac_config, layers_attr="mtp_layers")
    if compile_config is not None and compile_config.enable and "model" in compile_config.components:
        for name, block in list(model.layers.named_children()):
            if not getattr(block, "moe_enabled", False):
                # the sparse attention core and expert dispatch have data-dependent shapes: compile dense blocks only
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
