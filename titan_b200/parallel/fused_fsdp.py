"""Sharded linears whose FSDP collectives run inside the GEMM kernels (``parallelism.fsdp_fused_collectives``).

torch's FSDP2 all-gathers a parameter group, runs the layer, and reduce-scatters the gradients as separate NCCL
calls on side streams.  For the big linears this module does both inside compute kernels instead:

* forward   ``y = x · gather_rows(w_shard)ᵀ`` – `tb_ag_b_gemm`: copier CTAs pull every peer's weight shard once over
  NVLink into a local buffer while the tensor-core tiles that need only local rows already run;
* backward  ``dx = gy · W`` with the weight gathered again (one NCCL all-gather, overlapped with the wgrad GEMM),
  ``dW = gyᵀ · x`` on the tensor cores, then `tb_castscale_rs`: the gradient bucket is cast to fp32, scaled and
  reduce-scattered by peer loads in ONE kernel; each rank keeps only its ``[N/dp, K]`` slice.

The weight of a converted `nn.Linear` becomes a DTensor ``Shard(0)`` over the data-parallel mesh (the layout FSDP2 would
give it), so optimizers, gradient clipping and DCP checkpoints treat it like any FSDP parameter; FSDP2 itself is told
to ignore these parameters and keeps managing the rest (norms, embeddings).

Parity: the reference runs stock FSDP2 (`apply_fsdp`, torchtitan_npu/models/deepseek_v32/parallelize.py:236-262); this
is the fused counterpart for NVLink peers.
"""

from __future__ import annotations

import types

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.tensor import DTensor, Shard, distribute_tensor

from titan_b200.ops import fused_comm

__all__ = ["fused_fsdp_linear", "shard_linears", "FUSED_LINEAR_SUFFIXES"]

FUSED_LINEAR_SUFFIXES = ("attention.wq", "attention.wk", "attention.wv", "attention.wo", "feed_forward.w1",
                         "feed_forward.w2", "feed_forward.w3")


def _mm_nn(a, b):
    """a [M, N] · b [N, K] → [M, K]."""
    from titan_b200.ops import gemm as G

    if G.supported(a, b) and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0:
        return G.gemm(a.contiguous(), b.contiguous(), b_mn=True)
    return a @ b


def _mm_tn(a, b):
    from titan_b200.ops import gemm as G

    if G.supported(a, b) and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0:
        return G.gemm(a.contiguous(), b.contiguous(), a_mn=True, b_mn=True)
    return a.t() @ b


class _FusedFSDPLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_shard, group, grad_dtype):
        x2 = x.reshape(-1, x.shape[-1])
        y = fused_comm.all_gather_weight_matmul(x2, w_shard.to(x2.dtype), group)
        ctx.save_for_backward(x2, w_shard)
        ctx.group, ctx.shape, ctx.grad_dtype = group, x.shape, grad_dtype
        return y.reshape(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, gy):
        x2, w_shard = ctx.saved_tensors
        group = ctx.group
        world = dist.get_world_size(group)
        g2 = gy.reshape(-1, gy.shape[-1]).contiguous()
        w_full = torch.empty(world * w_shard.shape[0], w_shard.shape[1], dtype=x2.dtype, device=x2.device)
        work = dist.all_gather_into_tensor(w_full, w_shard.to(x2.dtype).contiguous(), group=group, async_op=True)
        dw_full = _mm_tn(g2, x2)                      # [N, K], runs while the weights arrive
        work.wait()
        dx = _mm_nn(g2, w_full)                       # [M, K]
        dw = fused_comm.castscale_reduce_scatter(dw_full.reshape(-1), 1.0, ctx.grad_dtype, group)
        return dx.reshape(ctx.shape), dw.view(w_shard.shape), None, None


def fused_fsdp_linear(x: torch.Tensor, w_shard: torch.Tensor, group, grad_dtype=None) -> torch.Tensor:
    """x [.., K]; w_shard [N/dp, K] (this rank's rows) → [.., N]; the weight gradient comes back as the local slice,
    summed over the group (the trainer normalises the loss by the global token count)."""
    return _FusedFSDPLinear.apply(x, w_shard, group, grad_dtype or w_shard.dtype)


def shard_linears(model: nn.Module, dp_mesh, suffixes=FUSED_LINEAR_SUFFIXES) -> list[nn.Parameter]:
    """Shard the weight rows of every matching `nn.Linear` over ``dp_mesh`` and route its forward through the fused
    kernels.  Returns the converted parameters (to be passed to FSDP2 as ``ignored_params``)."""
    group = dp_mesh.get_group()
    fused_comm.enable_for_group(group)
    world = dp_mesh.size()
    converted = []
    for name, mod in model.named_modules():
        if not isinstance(mod, nn.Linear) or not any(name.endswith(s) for s in suffixes) or mod.bias is not None:
            continue
        if mod.weight.shape[0] % world:
            continue
        if isinstance(mod.weight, DTensor):
            raise NotImplementedError("fused FSDP collectives compose with data parallelism only (no TP on the weight)")
        w = nn.Parameter(distribute_tensor(mod.weight.data, dp_mesh, [Shard(0)]), requires_grad=mod.weight.requires_grad)
        mod.register_parameter("weight", w)

        def fwd(self_, x, _group=group):
            return fused_fsdp_linear(x, self_.weight.to_local(), _group)

        mod.forward = types.MethodType(fwd, mod)
        converted.append(w)
    return converted
