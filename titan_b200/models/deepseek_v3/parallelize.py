"""Parallelisation of DeepSeek-V3: TP(+SP) for attention / dense FFN, CP (Ulysses on the SDPA core),
EP / ETP for experts, AC, compile, FSDP2 with experts on their own ``efsdp`` mesh.

Parity: torchtitan_npu/models/deepseek_v3/parallelize.py:23-82 (Ulysses CP + sequence-sharded MoE plan
on top of the upstream flow) and models/deepseek_v32/parallelize.py:127-284 for the overall order.
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
from titan_b200.parallel.tensor_parallel import NoParallel, maybe_enable_async_tp, parallelize_module

__all__ = ["parallelize_deepseekv3", "apply_non_moe_tp"]


def apply_non_moe_tp(model: nn.Module, tp_mesh, *, loss_parallel: bool) -> None:
    parallelize_module(model, tp_mesh, {
        "tok_embeddings": RowwiseParallel(input_layouts=Replicate(), output_layouts=Shard(1)),
        "norm": SequenceParallel(),
        "output": ColwiseParallel(input_layouts=Shard(1), output_layouts=Shard(-1) if loss_parallel else Replicate(),
                                  use_local_output=not loss_parallel),
    })
    for block in model.layers.values():
        attn = block.attention
        plan = {
            "attention_norm": SequenceParallel(),
            "attention": PrepareModuleInput(input_layouts=(Shard(1), None, None, None),
                                            desired_input_layouts=(Replicate(), None, None, None)),
            # the latent projections produce per-token latents shared by all heads: keep them replicated
            "attention.wkv_a": NoParallel(),
            "attention.kv_norm": NoParallel(),
            "attention.wkv_b": ColwiseParallel(),
            "attention.wo": RowwiseParallel(output_layouts=Shard(1)),
            "ffn_norm": SequenceParallel(),
        }
        if attn.q_lora_rank == 0:
            plan["attention.wq"] = ColwiseParallel()
        else:
            plan.update({"attention.wq_a": NoParallel(), "attention.q_norm": NoParallel(),
                         "attention.wq_b": ColwiseParallel()})
        if not block.moe_enabled:
            plan.update({
                "feed_forward": PrepareModuleInput(input_layouts=(Shard(1),), desired_input_layouts=(Replicate(),)),
                "feed_forward.w1": ColwiseParallel(),
                "feed_forward.w2": RowwiseParallel(output_layouts=Shard(1)),
                "feed_forward.w3": ColwiseParallel(),
            })
        parallelize_module(block, tp_mesh, plan)


def parallelize_deepseekv3(model: nn.Module, *, parallel_dims, training, model_converters=None, parallelism=None,
                           compile_config=None, ac_config=None, dump_folder: str = ""):
    pd = parallel_dims
    if training.seq_len % pd.seq_len_divisor != 0:
        raise ValueError(f"seq_len {training.seq_len} must be divisible by tp * 2 * cp = {pd.seq_len_divisor}")
    if pd.cp_enabled:
        n_heads = model.config.n_heads // (pd.tp if pd.tp_enabled else 1)
        if n_heads % pd.cp != 0:
            raise ValueError(f"Ulysses CP needs local heads ({n_heads}) divisible by cp ({pd.cp})")
    tp_mesh = pd.get_optional_mesh("tp")
    if tp_mesh is not None:
        maybe_enable_async_tp(parallelism, tp_mesh)
        apply_non_moe_tp(model, tp_mesh, loss_parallel=not parallelism.disable_loss_parallel)
    if pd.cp_enabled:
        from titan_b200.parallel.context_parallel import apply_cp_to_attention_module

        apply_cp_to_attention_module([b.attention.inner_attention for b in model.layers.values()],
                                     pd.get_mesh("cp"))
    if tp_mesh is not None or pd.ep_enabled:
        ep_mesh = pd.get_optional_mesh("ep")
        etp_mesh = pd.get_optional_mesh("etp") if pd.etp_enabled else None
        ep_etp = pd._sparse["ep", "etp"] if (pd.ep_enabled and pd.etp_enabled) else None
        apply_moe_ep_tp(model, tp_mesh=tp_mesh, ep_mesh=ep_mesh, etp_mesh=etp_mesh, ep_etp_mesh=ep_etp,
                        comm_backend=parallelism.expert_parallel_comm_backend)
    if ac_config is not None and ac_config.mode != "none":
        apply_ac(model, ac_config)
    if compile_config is not None and compile_config.enable and "model" in compile_config.components:
        for name, block in list(model.layers.named_children()):
            # routing produces data-dependent shapes: compile the dense parts only
            if not getattr(block, "moe_enabled", False):
                model.layers.register_module(name, torch.compile(block, backend=compile_config.backend))
    if pd.fsdp_enabled or pd.ep_enabled:
        names = ("dp_replicate", "fsdp") if pd.dp_replicate_enabled else None
        dp_mesh = pd.get_mesh(names) if names else pd.get_optional_mesh("fsdp")
        if dp_mesh is not None:
            edp = None
            if pd.ep_enabled:
                edp = pd.mesh_even_if_trivial("efsdp")  # a 1-rank efsdp mesh still isolates experts from the dense FSDP group
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
