"""Activation checkpointing: none / selective (op policy or every-Nth block) / full.

Selective-op mode keeps the outputs of expensive ops (matmuls, attention,
collectives, the fused sm_100a ops registered here) and recomputes the cheap
elementwise work.  Models may extend the save list for a scope with
`extend_sac_save_ops` (grouped-GEMM outputs in MoE blocks).

Parity: upstream `apply_ac` semantics plus the reference's save-list extension
context manager (torchtitan_npu/distributed/activation_checkpoint.py:20-42,
models/deepseek_v4/parallelize.py:368-383).
"""

from __future__ import annotations

import contextlib
from collections import defaultdict

import torch
import torch.nn as nn
from torch.distributed.algorithms._checkpoint.checkpoint_wrapper import checkpoint_wrapper
from torch.utils.checkpoint import CheckpointPolicy, create_selective_checkpoint_contexts

__all__ = ["apply_ac", "extend_sac_save_ops", "sac_save_ops", "register_sac_save_op"]

_aten = torch.ops.aten
_SAVE_OPS: set = {
    _aten.mm.default,
    _aten.addmm.default,
    _aten.bmm.default,
    _aten._scaled_dot_product_efficient_attention.default,
    _aten._scaled_dot_product_flash_attention.default,
    _aten._scaled_dot_product_cudnn_attention.default,
    _aten._scaled_dot_product_flash_attention_for_cpu.default,
    _aten.max.default,
}
for _name in ("reduce_scatter_tensor", "all_to_all_single", "all_gather_into_tensor"):
    _op = getattr(torch.ops._c10d_functional, _name, None)
    if _op is not None:
        _SAVE_OPS.add(_op.default)
if hasattr(_aten, "_grouped_mm"):
    _SAVE_OPS.add(_aten._grouped_mm.default)


def register_sac_save_op(op) -> None:
    """Fused custom ops call this at import so selective AC never recomputes them."""
    _SAVE_OPS.add(op)


def sac_save_ops() -> set:
    return set(_SAVE_OPS)


@contextlib.contextmanager
def extend_sac_save_ops(*ops):
    added = [op for op in ops if op not in _SAVE_OPS]
    _SAVE_OPS.update(added)
    try:
        yield
    finally:
        for op in added:
            _SAVE_OPS.discard(op)


def _op_policy(force_recompute_mm_shapes: set[tuple[int, ...]], save_every_mm: bool = False, extra_save_ops=()):
    """Per-op policy: attention, collectives and matmuls are saved, the rest is recomputed.  By default every
    SECOND matmul is recomputed (the memory-lean upstream rule); ``save_every_mm`` keeps them all: on a 180 GB part
    the extra ~0.75 GB per Llama-8B layer buys back one sixth of the step's GEMM work."""
    save_ops = set(_SAVE_OPS) | set(extra_save_ops)

    def make():
        meta = defaultdict(int)

        def policy(ctx, func, *args, **kwargs):
            if func == _aten.mm.default:
                if tuple(args[1].shape) in force_recompute_mm_shapes:
                    return CheckpointPolicy.PREFER_RECOMPUTE
                if save_every_mm:
                    return CheckpointPolicy.MUST_SAVE
                # save every second matmul: halves saved bytes, recompute stays cheap
                key = "recompute_mm" if ctx.is_recompute else "forward_mm"
                meta[key] += 1
                if meta[key] % 2 == 0:
                    return CheckpointPolicy.PREFER_RECOMPUTE
                return CheckpointPolicy.MUST_SAVE
            if func in save_ops:
                return CheckpointPolicy.MUST_SAVE
            return CheckpointPolicy.PREFER_RECOMPUTE

        return create_selective_checkpoint_contexts(policy)

    return make


def _wrap(module: nn.Module, ac_config, *, block_index: int, force_shapes: set) -> nn.Module:
    mode = ac_config.mode
    kw = dict(preserve_rng_state=ac_config.preserve_rng_state, determinism_check=ac_config.determinism_check,
              early_stop=ac_config.early_stop)
    if mode == "full":
        return checkpoint_wrapper(module, **kw)
    opt = str(ac_config.selective_ac_option)
    if opt in ("op", "op_save_all_mm"):
        extra = ()
        if getattr(ac_config, "selective_keep_swiglu", False):
            from titan_b200.ops.registry import SWIGLU_OPS

            extra = SWIGLU_OPS
        return checkpoint_wrapper(module, context_fn=_op_policy(force_shapes, save_every_mm=opt == "op_save_all_mm",
                                                                extra_save_ops=extra), **kw)
    if opt.isdigit():
        n = int(opt)
        if n <= 0:
            raise ValueError("selective_ac_option must be 'op', 'op_save_all_mm' or a positive integer")
        if block_index % n == 0:
            return checkpoint_wrapper(module, **kw)
        return module
    raise ValueError(f"invalid selective_ac_option {opt!r}")


def apply_ac(model: nn.Module, ac_config, *, layers_attr: str = "layers") -> None:
    """Wrap each transformer block of ``model.<layers_attr>`` in place."""
    if ac_config.mode == "none":
        return
    from titan_b200.ops import registry  # noqa: F401  (adds the sm_100a contraction ops to the save list)
    force_shapes: set[tuple[int, ...]] = set()
    for fqn in ac_config.per_op_sac_force_recompute_mm_shapes_by_fqns:
        for name, sub in model.named_modules():
            if name.endswith(fqn) and isinstance(sub, nn.Linear):
                force_shapes.add(tuple(sub.weight.t().shape))
    layers = getattr(model, layers_attr)
    for idx, (name, block) in enumerate(list(layers.named_children())):
        layers.register_module(name, _wrap(block, ac_config, block_index=idx, force_shapes=force_shapes))
