"""Parallelisation of the VLM: FSDP2 / HSDP data parallelism (per text block, per vision layer), AC on both towers.

Parity: torchtitan_npu/models/vlm/parallelize.py:18-55 (only data parallelism is supported; the recipe must name
the VLM converter).
"""

from __future__ import annotations

import torch.nn as nn

from titan_b200.parallel.activation_checkpoint import apply_ac
from titan_b200.parallel.fsdp import DTYPE_MAP, apply_fsdp, apply_replicate
from titan_b200.protocols.converter import has_converter

__all__ = ["parallelize_vlm"]


def _validate(parallel_dims, model_converters) -> None:
    pd = parallel_dims
    if pd.tp_enabled or pd.cp_enabled or pd.pp_enabled or pd.ep_enabled:
        raise NotImplementedError("the VLM currently only supports FSDP/HSDP data parallelism")
    convs = model_converters.converters if model_converters is not None else []
    if not has_converter(convs, "b200_vlm"):
        raise ValueError('the VLM requires "b200_vlm" in model_converters.converters')


def parallelize_vlm(model: nn.Module, *, parallel_dims, training, model_converters=None, parallelism=None,
                    compile_config=None, ac_config=None, dump_folder: str = ""):
    pd = parallel_dims
    _validate(pd, model_converters)
    if ac_config is not None and ac_config.mode != "none":
        apply_ac(model, ac_config)
        apply_ac(model.encoder, ac_config)
    if pd.fsdp_enabled:
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

        names = ("dp_replicate", "fsdp") if pd.dp_replicate_enabled else None
        dp_mesh = pd.get_mesh(names) if names else pd.get_mesh("fsdp")
        mp = MixedPrecisionPolicy(param_dtype=DTYPE_MAP[training.mixed_precision_param],
                                  reduce_dtype=DTYPE_MAP[training.mixed_precision_reduce])
        for layer in model.encoder.layers.values():  # the vision tower gets its own units, then one for its rest
            fully_shard(layer, mesh=dp_mesh, mp_policy=mp)
        fully_shard(model.encoder, mesh=dp_mesh, mp_policy=mp)
        fully_shard(model.projector, mesh=dp_mesh, mp_policy=mp)
        apply_fsdp(model, dp_mesh, param_dtype=DTYPE_MAP[training.mixed_precision_param],
                   reduce_dtype=DTYPE_MAP[training.mixed_precision_reduce], pp_enabled=False,
                   cpu_offload=training.enable_cpu_offload,
                   reshard_after_forward_policy=parallelism.fsdp_reshard_after_forward,
            reduce_scatter=parallelism.fsdp_reduce_scatter,
            all_gather=parallelism.fsdp_all_gather)
    elif pd.dp_replicate_enabled:
        apply_replicate(model, pd.get_mesh(("dp_replicate", "fsdp")), param_dtype=DTYPE_MAP[training.mixed_precision_param],
                        reduce_dtype=DTYPE_MAP[training.mixed_precision_reduce])
    return model
