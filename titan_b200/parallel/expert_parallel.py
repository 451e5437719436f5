"""Expert-parallel styles for `GroupedExperts`.

* `ExpertParallel`        – experts sharded on dim 0 over the ``ep`` mesh; tokens travel by
  all-to-all (NCCL baseline): count exchange → token all-to-all → rank-major → local-expert-major
  re-routing; the output hook reverses all three.
* `FusedExpertParallel`   – same placement; dispatch/combine run as ONE kernel each over peer
  memory (`titan_b200.ops.moe_comm`): rows are written straight into the owner's expert-major buffer.
* `ExpertTensorParallel`  – 2-D ``[ep, etp]``: dim 0 over ep, ``w1/w3`` dim 1 and ``w2`` dim 2 over etp.
* `TensorParallel`        – every rank sees all tokens, weights split over ``tp`` on the hidden dim.

Both tensor-parallel styles leave the routed output as a PARTIAL sum over the tp / etp ranks: the MoE block
declares its output ``Partial()`` and the reduce-scatter back to the sequence shard adds the ranks up once.  In
backward the gradient of the (replicated) routed input is the matching partial sum and is all-reduced where the
tokens enter the experts.  A fused ``w13 = [w1 | w3]`` weight is split so that every rank holds
``[w1_shard | w3_shard]`` (the layout `checkpoint.weight_utils` fuses and splits).
* `permute / unpermute`   – the local re-routing used by the dispatch and by the single-process dry run.

Under a fake process group the result of the count exchange is meaningless, so splits are taken
from the local counts (every rank is assumed to send what it receives).

Parity: upstream `ExpertParallel / TensorParallel / ExpertTensorParallel / _permute / _unpermute`
and the reference's variants (torchtitan_npu/converters/kernels/moe_dispatch.py:155-287,
patches/torchtitan/expert_parallel.py:27-184, converters/kernels/permutation.py:57-143).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed._functional_collectives import all_to_all_single, all_to_all_single_autograd
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.tensor import DTensor, Shard, distribute_module, distribute_tensor
from torch.distributed.tensor.parallel import ParallelStyle

from titan_b200.parallel.fake_pg import is_fake_process_group

__all__ = ["ExpertParallel", "FusedExpertParallel", "ExpertTensorParallel", "TensorParallel", "permute", "unpermute",
           "rerouting_indices"]


def rerouting_indices(counts_by_rank_expert: torch.Tensor) -> torch.Tensor:
    """Row permutation rank-major → local-expert-major for ``counts[ep, E_local]`` (tokens per
    (source rank, local expert)).  Output position i holds the rank-major row that belongs there."""
    ep, e_local = counts_by_rank_expert.shape
    c = counts_by_rank_expert.reshape(-1).long()
    starts = torch.cumsum(c, 0) - c  # start of each (rank, expert) chunk in the received buffer
    chunk_order = torch.arange(ep * e_local, device=c.device).view(ep, e_local).t().reshape(-1)
    lens = c[chunk_order]
    total = int(lens.sum())
    if total == 0:
        return torch.empty(0, dtype=torch.long, device=c.device)
    out_starts = torch.cumsum(lens, 0) - lens
    chunk_id = torch.repeat_interleave(torch.arange(ep * e_local, device=c.device), lens, output_size=total)
    within = torch.arange(total, device=c.device) - out_starts[chunk_id]
    return starts[chunk_order][chunk_id] + within


def permute(x: torch.Tensor, counts_by_rank_expert: torch.Tensor):
    idx = rerouting_indices(counts_by_rank_expert)
    return x[idx], idx


def unpermute(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    out[idx] = x
    return out


class ExpertParallel(ParallelStyle):
    def __init__(self):
        super().__init__()
        self.input_splits = self.output_splits = None
        self.perm = None
        self.input_shape = None

    @staticmethod
    def _partition_fn(name, mod, device_mesh):
        for pname, p in list(mod.named_parameters(recurse=False)):
            mod.register_parameter(pname, nn.Parameter(distribute_tensor(p, device_mesh, [Shard(0)])))

    def _splits(self, counts: torch.Tensor, group, ep: int):
        """→ (counts_by_src_rank_local_expert [ep, E_local], input_splits, output_splits) with one D2H sync."""
        if is_fake_process_group(group):
            grouped = counts.view(ep, -1)
            in_s = grouped.sum(1).long().tolist()
            return grouped, in_s, list(in_s)
        with torch.no_grad():
            recv = all_to_all_single(counts, None, None, group=group)
            recv = torch.ops._c10d_functional.wait_tensor(recv)
            both = torch.stack([counts.view(ep, -1).sum(1), recv.view(ep, -1).sum(1)]).long().cpu()
        return recv.view(ep, -1), both[0].tolist(), both[1].tolist()

    def _token_dispatch(self, mod, inputs, device_mesh):
        routed_input, num_tokens_per_expert = inputs
        ep = device_mesh.size()
        group = device_mesh.get_group()
        counts = num_tokens_per_expert.to(torch.int64 if not routed_input.is_cuda else torch.int64)
        grouped, self.input_splits, self.output_splits = self._splits(counts, group, ep)
        self.input_shape = routed_input.shape
        if is_fake_process_group(group):
            received = routed_input
        else:
            received = all_to_all_single_autograd(routed_input, self.output_splits, self.input_splits, group)
        received, self.perm = permute(received, grouped)
        return received, grouped.sum(0)

    def _token_combine(self, mod, routed_output, device_mesh):
        group = device_mesh.get_group()
        routed_output = _unpermute_autograd(routed_output, self.perm)
        if is_fake_process_group(group):
            return routed_output
        return all_to_all_single_autograd(routed_output, self.input_splits, self.output_splits, group)

    def _apply(self, module: nn.Module, device_mesh: DeviceMesh) -> nn.Module:
        return distribute_module(module, device_mesh, partition_fn=self._partition_fn,
                                 input_fn=self._token_dispatch, output_fn=self._token_combine)


class _Unpermute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx):
        ctx.save_for_backward(idx)
        return unpermute(x, idx)

    @staticmethod
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        return g[idx], None


def _unpermute_autograd(x, idx):
    return _Unpermute.apply(x, idx)


class FusedExpertParallel(ExpertParallel):
    """Same sharding as `ExpertParallel`; tokens move through the peer-memory dispatch / combine kernels.

    The fused MoE layer (`b200_moe_dispatch`) drives the exchange itself from its device-side routing plan, so
    this style only shards the expert weights and records the mesh on the module.  Experts that were not
    converted keep the NCCL hooks of the parent class."""

    def _apply(self, module: nn.Module, device_mesh: DeviceMesh) -> nn.Module:
        if not hasattr(module, "forward_padded"):
            return super()._apply(module, device_mesh)
        module = distribute_module(module, device_mesh, partition_fn=self._partition_fn)
        module.ep_mesh = device_mesh
        return module


def _shard_hidden(pname: str, p: torch.Tensor, device_mesh, lead: tuple = ()):
    """Placement of one expert weight under (expert) tensor parallelism: ``w1 / w3 / w13`` on the hidden rows
    (dim 1), ``w2`` on its hidden columns (dim 2); ``lead`` are the placements of leading mesh axes (EP)."""
    if pname == "w13":
        # [E, 2H, D] holds w1 above w3: every rank takes its rows of BOTH halves
        w1, w3 = p.data.chunk(2, dim=1)
        l1 = distribute_tensor(w1, device_mesh, [*lead, Shard(1)]).to_local()
        l3 = distribute_tensor(w3, device_mesh, [*lead, Shard(1)]).to_local()
        local = torch.cat([l1, l3], dim=1)
        return DTensor.from_local(local, device_mesh, [*lead, Shard(1)], run_check=False, shape=p.shape,
                                  stride=p.stride())
    dim = 2 if pname == "w2" else 1
    return distribute_tensor(p, device_mesh, [*lead, Shard(dim)])


class _AllReduceGrad(torch.autograd.Function):
    """Identity whose gradient is summed over ``group`` (a replicated input consumed by per-rank weight shards)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class TensorParallel(ParallelStyle):
    """Experts see all tokens; ``w1/w3`` are split on the hidden dim (1), ``w2`` on its input dim (2).  The output
    stays a partial sum over the mesh (see the module docstring)."""

    @staticmethod
    def _partition_fn(name, mod, device_mesh):
        for pname, p in list(mod.named_parameters(recurse=False)):
            if p is None:
                continue
            mod.register_parameter(pname, nn.Parameter(_shard_hidden(pname, p, device_mesh)))

    @staticmethod
    def _input_fn(mod, inputs, device_mesh):
        x = inputs[0]
        if isinstance(x, torch.Tensor) and x.requires_grad:
            x = _AllReduceGrad.apply(x, device_mesh.get_group())
        return (x, *inputs[1:])

    def _apply(self, module, device_mesh):
        return distribute_module(module, device_mesh, partition_fn=self._partition_fn, input_fn=self._input_fn)


class ExpertTensorParallel(ExpertParallel):
    """2-D mesh ``[ep, etp]``: EP on dim 0, TP on the hidden dim."""

    def _token_dispatch(self, mod, inputs, device_mesh):
        x = inputs[0]
        if x.requires_grad:  # every etp rank dispatches the same tokens to its own hidden slice of the experts
            x = _AllReduceGrad.apply(x, device_mesh["etp"].get_group())
        return super()._token_dispatch(mod, (x, *inputs[1:]), device_mesh["ep"])

    def _token_combine(self, mod, routed_output, device_mesh):
        return super()._token_combine(mod, routed_output, device_mesh["ep"])  # partial over etp

    @staticmethod
    def _partition_fn_2d(name, mod, device_mesh):
        for pname, p in list(mod.named_parameters(recurse=False)):
            if p is None:
                continue
            mod.register_parameter(pname, nn.Parameter(_shard_hidden(pname, p, device_mesh, (Shard(0),))))

    def _apply(self, module, device_mesh):
        return distribute_module(module, device_mesh, partition_fn=self._partition_fn_2d,
                                 input_fn=self._token_dispatch, output_fn=self._token_combine)
