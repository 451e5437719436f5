"""Parallelisation of DeepSeek-V4: TP/SP, compressed-attention CP, EP, AC, FSDP2, indexer-loss tracking.

Tensor-parallel layout (activations between modules are plain local tensors):

* the ``hc`` residual streams stay sequence-sharded ``[B, S/tp, hc, D]`` through the whole block: `hc_pre`,
  `hc_post` and the stream-collapsing heads are token-local, so they run on the local shard without any
  collective; their replicated fp32 mixing parameters collect partial gradients that are summed over the mesh;
* the attention input is gathered along the sequence; the latent projections (``wq_a, q_norm, wkv, kv_norm``),
  both compressors and the whole indexer are replicated computations; ``wq_b`` is column-parallel (heads split),
  ``attn_sink`` is split by head, ``wo_a`` is split by output group and ``wo_b`` is row-parallel with a
  reduce-scatter back to the sequence shard;
* the attention core sees local heads and the replicated KV latents: the gradients of ``kv`` and ``kv_compress``
  are partial sums and are all-reduced in backward; the indexer's teacher distribution is summed over the ranks'
  heads with one small all-reduce;
* MoE: tokens gathered for routing, outputs reduce-scattered (shared plan), token ids pass through for hash routing.

Parity: torchtitan_npu/models/deepseek_v4/parallelize.py:141-1099.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch.distributed.tensor import Replicate, Shard, distribute_tensor
from torch.distributed.tensor.parallel import (
    ColwiseParallel,
    PrepareModuleInput,
    RowwiseParallel,
    SequenceParallel,
)

from titan_b200.models.common.dsa_indexer_loss import DSAIndexerLossAutoScaler
from titan_b200.models.deepseek_v32.parallelize import apply_distributed_indexer_loss_tracking
from titan_b200.parallel.activation_checkpoint import apply_ac
from titan_b200.parallel.fsdp import DTYPE_MAP, apply_fsdp, apply_replicate
from titan_b200.parallel.moe_parallelize import apply_moe_ep_tp
from titan_b200.parallel.tensor_parallel import (
    AwaitRowwiseParallel,
    NoParallel,
    PrepareModuleInputOutputWithBwdAllReduce,
    SequenceShardedLinear,
    maybe_enable_async_tp,
    parallelize_module,
)
from titan_b200.protocols.converter import has_converter
from titan_b200.utils.logging import logger

__all__ = ["parallelize_deepseekv4", "apply_non_moe_tp", "validate_parallelism"]

_HC_PARAMS = ("hc_attn_fn", "hc_ffn_fn", "hc_attn_base", "hc_ffn_base", "hc_attn_scale", "hc_ffn_scale")
_HEAD_PARAMS = ("hc_head_fn", "hc_head_base", "hc_head_scale")


def _distribute_param(module: nn.Module, name: str, mesh, placements) -> None:
    p = getattr(module, name)
    setattr(module, name, nn.Parameter(distribute_tensor(p.data, mesh, placements), requires_grad=p.requires_grad))


def validate_parallelism(cfg, parallel_dims, converters) -> None:
    if parallel_dims.tp_enabled:
        tp = parallel_dims.tp
        if cfg.n_heads % tp or cfg.o_groups % tp:
            raise ValueError(f"tensor parallel degree {tp} must divide n_heads {cfg.n_heads} and o_groups "
                             f"{cfg.o_groups}")
    if parallel_dims.cp_enabled and not has_converter(converters, "b200_smla"):
        raise NotImplementedError("context parallelism for DeepSeek-V4 runs on the fused sparse attention only: "
                                  "add the `b200_smla` converter")
    if parallel_dims.pp_enabled and cfg.num_mtp_modules > 0:
        raise NotImplementedError("DeepSeek-V4 MTP with pipeline parallelism is not supported")


def apply_non_moe_tp(model: nn.Module, tp_mesh, *, loss_parallel: bool) -> None:
    root = {}
    if getattr(model, "tok_embeddings", None) is not None:
        root["tok_embeddings"] = RowwiseParallel(input_layouts=Replicate(), output_layouts=Shard(1))
    if getattr(model, "norm", None) is not None:
        root["norm"] = SequenceParallel()
    if getattr(model, "output", None) is not None:
        root["output"] = ColwiseParallel(input_layouts=Shard(1),
                                         output_layouts=Shard(-1) if loss_parallel else Replicate(),
                                         use_local_output=not loss_parallel)
    if root:
        parallelize_module(model, tp_mesh, root)
    group = tp_mesh.get_group()
    for block in model.layers.values():
        if block is None:
            continue
        for name in _HC_PARAMS:
            _distribute_param(block, name, tp_mesh, [Replicate()])
        inner, pre = block.attention.inner_attention, block.attention.pre_attention
        _distribute_param(inner, "attn_sink", tp_mesh, [Shard(0)])
        inner.tp_group = group
        plan = {
            "attention_norm": SequenceParallel(use_local_output=True),
            "attention": PrepareModuleInput(input_layouts=(Shard(1), None, None, None),
                                            desired_input_layouts=(Replicate(), None, None, None),
                                            use_local_output=True),
            "attention.pre_attention.wq_a": NoParallel(),
            "attention.pre_attention.q_norm": NoParallel(),
            "attention.pre_attention.wq_b": ColwiseParallel(),
            "attention.pre_attention.wkv": NoParallel(),
            "attention.pre_attention.kv_norm": NoParallel(),
            # kv (arg 1) and kv_compress (arg 2) are replicated latents read by every rank's heads
            "attention.inner_attention": PrepareModuleInputOutputWithBwdAllReduce(
                bwd_allreduce_input_idx=(1, 2), input_layouts=None, desired_input_layouts=None,
                output_layouts=None, desired_output_layouts=None),
            "attention.post_attention.wo_a": ColwiseParallel(),  # never called: only shards the groups
            "attention.post_attention.wo_b": AwaitRowwiseParallel(output_layouts=Shard(1)),
            "ffn_norm": SequenceParallel(use_local_output=True),
        }
        compressors = []
        for attr in ("compressor", "compressor_128"):
            if hasattr(pre, attr):
                compressors.append((f"attention.pre_attention.{attr}", getattr(pre, attr)))
        if hasattr(pre, "indexer"):
            plan["attention.pre_attention.indexer.wq_b"] = NoParallel()
            plan["attention.pre_attention.indexer.weights_proj"] = NoParallel()
            compressors.append(("attention.pre_attention.indexer.compressor", pre.indexer.compressor))
        for key, comp in compressors:
            _distribute_param(comp, "ape", tp_mesh, [Replicate()])
            plan[f"{key}.wkv"] = NoParallel()
            plan[f"{key}.wgate"] = NoParallel()
            plan[f"{key}.norm"] = NoParallel()
        if getattr(block, "is_last_layer", False):
            for name in _HEAD_PARAMS:
                _distribute_param(block.hc_head, name, tp_mesh, [Replicate()])
        if hasattr(block, "mtp_hc_head"):
            for name in _HEAD_PARAMS:
                _distribute_param(block.mtp_hc_head, name, tp_mesh, [Replicate()])
            plan.update({"enorm": SequenceParallel(use_local_output=True),
                         "hnorm": SequenceParallel(use_local_output=True),
                         "e_proj": SequenceShardedLinear(),
                         "h_proj": SequenceShardedLinear(),
                         "mtp_norm": SequenceParallel(use_local_output=True)})
        parallelize_module(block, tp_mesh, plan)


def apply_compile(model: nn.Module, compile_config, *, use_global_tnd: bool = False) -> int:
    """Per-submodule compile plan (opt-in, `--compile.enable`): inside every block the projections around the attention
    core (`pre_attention`, `post_attention`) and the MoE's router and shared experts are compiled in place; the
    attention core and the routed experts are not (hand-written kernels with data-dependent shapes, and the experts
    carry FSDP hooks that a compiled region must not swallow), nor are the norms (kernel converters) and the
    hyper-connection mixing, which the block runs itself.  With packed streams (`use_global_tnd`) the stream layout
    is data dependent in `pre_attention`, which then stays eager as well.  `nn.Module.compile` keeps the module
    objects, so parameter names and checkpoints do not change.  Returns the number of compiled submodules.

    Parity: torchtitan_npu/models/deepseek_v4/parallelize.py:958-1044 (compile around the experts' hooks, skip the
    inner attention, the hyper-connection pre step and the fused norms)."""
    skip = {"attention": {"inner_attention"} | ({"pre_attention"} if use_global_tnd else set()), "moe": {"experts"}}
    count = 0
    for block in model.layers.values():
        if block is None:
            continue
        inner = getattr(block, "_checkpoint_wrapped_module", block)
        for parent_name, skipped in skip.items():
            parent = getattr(inner, parent_name, None)
            if parent is None:
                continue
            for name, child in parent.named_children():
                if name in skipped or "norm" in type(child).__name__.lower():
                    continue
                child.compile(backend=compile_config.backend, fullgraph=False)
                count += 1
    return count


def parallelize_deepseekv4(model: nn.Module, *, parallel_dims, training, model_converters=None, parallelism=None,
                           compile_config=None, ac_config=None, dump_folder: str = ""):
    pd = parallel_dims
    cfg = model.config
    if training.seq_len % pd.seq_len_divisor != 0:
        raise ValueError(f"seq_len {training.seq_len} must be divisible by tp * 2 * cp = {pd.seq_len_divisor}")
    convs = model_converters.converters if model_converters is not None else []
    validate_parallelism(cfg, pd, convs)
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
        from titan_b200.parallel.context_parallel import compressor_attention_cp  # noqa: F401  (registers)

        apply_cp_to_attention_module([b.attention for b in model.layers.values() if b is not None],
                                     pd.get_mesh("cp"))
    if tp_mesh is not None or pd.ep_enabled:
        ep_etp = pd._sparse["ep", "etp"] if (pd.ep_enabled and pd.etp_enabled) else None
        apply_moe_ep_tp(model, tp_mesh=tp_mesh, ep_mesh=pd.get_optional_mesh("ep"),
                        etp_mesh=pd.get_optional_mesh("etp") if pd.etp_enabled else None, ep_etp_mesh=ep_etp,
                        comm_backend=parallelism.expert_parallel_comm_backend, extra_moe_inputs=1)
    if ac_config is not None and ac_config.mode != "none":
        apply_ac(model, ac_config)
    if compile_config is not None and compile_config.enable and "model" in compile_config.components:
        n = apply_compile(model, compile_config, use_global_tnd=bool(getattr(model.config, "use_global_tnd", False)))
        logger.info("compiled %d DeepSeek-V4 submodules around the attention cores and the experts", n)
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
