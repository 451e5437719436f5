"""Tensor-parallel helpers shared by all models.

* `parallelize_module` – the entry point every model plan goes through; active
  converter plan-updaters may rewrite the plan first (e.g. swap the NCCL
  expert-parallel style for the fused peer-memory one).
* `NoParallel` – keeps a module replicated but makes its params DTensors on the
  TP mesh so gradient clipping / DCP see a uniform layout.
* `AwaitRowwiseParallel` – row-parallel style whose output is waited on before
  leaving the module (an un-awaited async collective tensor leaks under AC).
* `PrepareModuleInputOutputWithBwdAllReduce` – replicated inputs to an attention
  kernel whose gradients must be summed over TP.
* `maybe_enable_async_tp` – selects the fused all-gather→GEMM / GEMM→reduce-scatter
  kernels for sequence-parallel linears.

Parity: torchtitan_npu/converters/framework/parallelize_plan_update_wrapper.py:24-48,
models/deepseek_v32/parallelize.py:57-124, patches/torch/micro_pipeline_tp.py:114-144.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.tensor import DTensor, Replicate, Shard, distribute_module, distribute_tensor
from torch.distributed.tensor.parallel import (
    ParallelStyle,
    PrepareModuleInputOutput,
    RowwiseParallel,
)
from torch.distributed.tensor.parallel import parallelize_module as _torch_parallelize_module

from titan_b200.protocols.converter import active_plan_updaters

__all__ = [
    "parallelize_module",
    "NoParallel",
    "AwaitRowwiseParallel",
    "PrepareModuleInputOutputWithBwdAllReduce",
    "SequenceShardedLinear",
    "FusedRowwiseParallel",
    "ReplicateParams",
    "norm_weight_local",
    "replicated_param_local",
    "maybe_enable_async_tp",
    "async_tp_enabled",
]

_ASYNC_TP = {"enabled": False}


def parallelize_module(module: nn.Module, device_mesh: DeviceMesh | None = None, parallelize_plan=None, **kwargs):
    for updater in active_plan_updaters():
        parallelize_plan = updater.update(parallelize_plan)
    if _ASYNC_TP["enabled"] and isinstance(parallelize_plan, dict):
        # async tensor parallelism, model-independent half: every row-parallel linear whose output goes back to the
        # sequence shard runs its reduce-scatter inside the GEMM (any model plan; embeddings and biased linears keep
        # their original style)
        parallelize_plan = {k: (FusedRowwiseParallel(v) if _is_seq_rowwise(v) else v)
                            for k, v in parallelize_plan.items()}
    return _torch_parallelize_module(module, device_mesh, parallelize_plan, **kwargs)


def _is_seq_rowwise(style) -> bool:
    return (type(style) in (RowwiseParallel, AwaitRowwiseParallel)
            and tuple(getattr(style, "output_layouts", ())) == (Shard(1),)
            and tuple(getattr(style, "input_layouts", ())) == (Shard(-1),)
            and getattr(style, "use_local_output", True))


class NoParallel(ParallelStyle):
    def __init__(self, *, input_layout=None, output_layout=None, use_local_output: bool = True):
        super().__init__()
        self.input_layout = input_layout or Replicate()
        self.output_layout = output_layout or Replicate()
        self.desired_input_layout = Replicate()
        self.use_local_output = use_local_output

    @staticmethod
    def _prepare_input_fn(input_layout, desired_input_layout, mod, inputs, device_mesh):
        x = inputs[0]
        if not isinstance(x, DTensor):
            x = DTensor.from_local(x, device_mesh, (input_layout,), run_check=False)
        if (input_layout,) != (desired_input_layout,):
            x = x.redistribute(placements=(desired_input_layout,), async_op=True)
        return (x, *inputs[1:])

    @staticmethod
    def _prepare_output_fn(output_layout, use_local_output, mod, outputs, device_mesh):
        if outputs.placements != (output_layout,):
            outputs = outputs.redistribute(placements=(output_layout,), async_op=True)
        return outputs.to_local(grad_placements=(output_layout,)) if use_local_output else outputs

    def _apply(self, module: nn.Module, device_mesh: DeviceMesh) -> nn.Module:
        from functools import partial

        return distribute_module(
            module,
            device_mesh,
            None,
            partial(self._prepare_input_fn, self.input_layout, self.desired_input_layout),
            partial(self._prepare_output_fn, self.output_layout, self.use_local_output),
        )


class AwaitRowwiseParallel(RowwiseParallel):
    @staticmethod
    def _prepare_output_fn(output_layouts, use_local_output, mod, outputs, device_mesh):
        out = RowwiseParallel._prepare_output_fn(output_layouts, use_local_output, mod, outputs, device_mesh)
        if isinstance(out, torch.Tensor) and not isinstance(out, DTensor):
            out = torch.ops._c10d_functional.wait_tensor(out) if type(out).__name__ == "AsyncCollectiveTensor" else out
        return out


class _AllReduceBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


class PrepareModuleInputOutputWithBwdAllReduce(ParallelStyle):
    """Sums the grads of the inputs listed in ``bwd_allreduce_input_idx`` over the mesh: each TP rank attends
    with its own heads to the same replicated K/V latent, so dK/dV are partial sums.

    With layouts given it also behaves like `PrepareModuleInputOutput`; with ``input_layouts=None`` the module's
    inputs and outputs are plain local tensors and are left alone."""

    def __init__(self, *, bwd_allreduce_input_idx: tuple[int, ...] = (), input_layouts=None,
                 desired_input_layouts=None, output_layouts=None, desired_output_layouts=None, **kwargs):
        super().__init__()
        self.bwd_allreduce_input_idx = tuple(bwd_allreduce_input_idx)
        self.inner = None
        if input_layouts is not None or output_layouts is not None:
            self.inner = PrepareModuleInputOutput(
                input_layouts=input_layouts, desired_input_layouts=desired_input_layouts,
                output_layouts=output_layouts, desired_output_layouts=desired_output_layouts, **kwargs)

    def _apply(self, module: nn.Module, device_mesh: DeviceMesh) -> nn.Module:
        if self.inner is not None:
            module = self.inner._apply(module, device_mesh)
        group = device_mesh.get_group()
        idxs = self.bwd_allreduce_input_idx

        def pre_hook(mod, args):
            args = list(args)
            for i in idxs:
                if i < len(args) and isinstance(args[i], torch.Tensor) and args[i].requires_grad:
                    args[i] = _AllReduceBwd.apply(args[i], group)
            return tuple(args)

        module.register_forward_pre_hook(pre_hook)
        return module


def replicated_param_local(p, *, partial_grad: bool):
    """Local tensor of a parameter that is replicated over its mesh.  ``partial_grad``: the parameter is applied to
    activations that differ per rank (sequence-sharded), so its gradient is summed over the mesh in backward."""
    if not isinstance(p, DTensor):
        return p
    local = p.to_local()
    if partial_grad:
        local = _AllReduceBwd.apply(local, p.device_mesh.get_group())
    return local


def norm_weight_local(w, x):
    """Local weight of a norm whose parameter is replicated over a mesh.  The gradient is complete on every rank only
    if the activations are replicated too (a `Replicate` DTensor); sharded DTensors and plain local tensors (per-rank
    heads or sequence slices) leave a partial sum that is reduced in backward."""
    if not isinstance(w, DTensor):
        return w
    replicated = isinstance(x, DTensor) and all(isinstance(pl, Replicate) for pl in x.placements)
    return replicated_param_local(w, partial_grad=not replicated)


class ReplicateParams(ParallelStyle):
    """Only turns the module's parameters into replicated DTensors (uniform layout for clipping / checkpoints); the
    module itself keeps working on local tensors."""

    def _apply(self, module: nn.Module, device_mesh: DeviceMesh) -> nn.Module:
        for name, p in list(module.named_parameters(recurse=False)):
            module.register_parameter(name, nn.Parameter(distribute_tensor(p.data, device_mesh, [Replicate()]),
                                                         requires_grad=p.requires_grad))
        return module


class ShardOnly(ParallelStyle):
    """Shard a linear's weight along ``dim`` (0 = column-parallel / output features, 1 = row-parallel / input
    features) and nothing else: no input or output hooks.  The module's forward is provided by the fused
    sequence-parallel path, which reads the local shard itself."""

    def __init__(self, dim: int):
        super().__init__()
        self.dim = dim

    def _apply(self, module: nn.Module, device_mesh: DeviceMesh) -> nn.Module:
        for name, p in list(module.named_parameters(recurse=False)):
            placement = Shard(self.dim) if p.dim() > self.dim else Replicate()
            module.register_parameter(name, nn.Parameter(distribute_tensor(p.data, device_mesh, [placement]),
                                                         requires_grad=p.requires_grad))
        return module


class FusedRowwiseParallel(ParallelStyle):
    """`RowwiseParallel(output_layouts=Shard(1))` with the reduce-scatter fused into the GEMM: the weight keeps its
    input-feature shard, the forward multiplies the local activations and the epilogue of the GEMM stores every tile
    into the staging slot of the rank that owns those sequence rows (`titan_b200.parallel.async_tp.linear_rs`).
    [batch, sequence, features] inputs take the fused kernel, one launch per sequence; other shapes, biased linears
    and non-linear modules (the embedding) fall back to the wrapped style or to a library reduce-scatter with the same result."""

    def __init__(self, fallback: ParallelStyle):
        super().__init__()
        self.fallback = fallback

    def _apply(self, module: nn.Module, device_mesh: DeviceMesh) -> nn.Module:
        if not isinstance(module, nn.Linear) or module.bias is not None:
            return self.fallback._apply(module, device_mesh)
        from torch.distributed.tensor import Partial

        module.register_parameter("weight", nn.Parameter(
            distribute_tensor(module.weight.data, device_mesh, [Shard(1)]), requires_grad=module.weight.requires_grad))
        group = device_mesh.get_group()

        def forward(x, _m=module):
            from titan_b200.parallel.async_tp import linear_rs_batched

            w = _m.weight.to_local()
            if isinstance(x, DTensor):
                x = x.to_local()
            if x.dim() == 3:
                return linear_rs_batched(x.to(w.dtype), w, group)   # one fused launch per sequence
            y = torch.nn.functional.linear(x, w)
            return DTensor.from_local(y, device_mesh, [Partial()]).redistribute(placements=[Shard(1)]).to_local()

        module.forward = forward
        module._async_tp = "gemm_reduce_scatter"
        return module


class SequenceShardedLinear(ParallelStyle):
    """A full (unsplit) linear applied to sequence-sharded local activations: the weight is replicated, every rank
    multiplies its own tokens, and the weight gradient is a partial sum that is reduced over the mesh."""

    def _apply(self, module: nn.Module, device_mesh: DeviceMesh) -> nn.Module:
        from torch.distributed.tensor import Partial

        for name, p in list(module.named_parameters(recurse=False)):
            module.register_parameter(name, nn.Parameter(distribute_tensor(p.data, device_mesh, [Replicate()]),
                                                         requires_grad=p.requires_grad))

        def forward(x, _m=module):
            w = replicated_param_local(_m.weight, partial_grad=True)
            b = replicated_param_local(_m.bias, partial_grad=True) if _m.bias is not None else None
            return torch.nn.functional.linear(x, w, b)

        module.forward = forward
        return module


def maybe_enable_async_tp(parallelism_config, tp_mesh: DeviceMesh | None) -> bool:
    """Turn on the fused SP kernels when requested; returns whether they are on."""
    if tp_mesh is None or not getattr(parallelism_config, "enable_async_tensor_parallel", False):
        _ASYNC_TP["enabled"] = False
        return False
    from titan_b200.ops import fused_comm

    if not torch.cuda.is_available():
        # same dataflow through the library fallbacks of the fused ops (fp32 on CPU): used to test the autograd logic
        import warnings

        warnings.warn("enable_async_tensor_parallel without CUDA: the fused kernels fall back to library collectives")

    fused_comm.enable_for_group(tp_mesh.get_group())
    _ASYNC_TP["enabled"] = True
    return True


def async_tp_enabled() -> bool:
    return _ASYNC_TP["enabled"]
