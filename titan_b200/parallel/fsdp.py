"""FSDP2 / HSDP / replicate wrapping.

Per-block `fully_shard` with a mixed-precision policy (bf16 params/compute,
fp32 reduce by default).  Experts are sharded on their own ``efsdp`` mesh when
expert parallelism is on, and every group divides gradients by the same factor.

With ``fused_collectives=True`` the per-block parameter all-gather is replaced
by the peer-memory path: shards are published in symmetric memory and the first
consuming GEMM of the block reads them tile by tile
(`titan_b200.ops.fused_comm.fsdp_allgather_gemm`); gradients go through the
cast+scale+reduce-scatter kernel.  Without it, NCCL all-gather / reduce-scatter
issued by FSDP2 are used (the baseline the fused path is measured against).

Parity: upstream `apply_fsdp(model, dp_mesh, param_dtype, reduce_dtype,
pp_enabled, cpu_offload, reshard_after_forward_policy, ep_degree, edp_mesh,
gradient_divide_factor)` and `apply_replicate` as used by the reference
(torchtitan_npu/models/deepseek_v32/parallelize.py:255-294,
models/deepseek_v4/parallelize.py:202-254,435-450).
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.fsdp import CPUOffloadPolicy, MixedPrecisionPolicy, fully_shard

__all__ = ["apply_fsdp", "apply_replicate", "DTYPE_MAP", "reshard_policy"]

DTYPE_MAP = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def reshard_policy(policy: str, pp_enabled: bool) -> bool:
    if policy == "always":
        return True
    if policy == "never":
        return False
    if policy == "default":
        # under PP each microbatch would re-gather; keep params unsharded between fwd and bwd
        return not pp_enabled
    raise ValueError(f"invalid fsdp_reshard_after_forward {policy!r}")


def _blocks(model: nn.Module, layers_attr: str):
    layers = getattr(model, layers_attr, None)
    if layers is None:
        return []
    return [(n, b) for n, b in layers.named_children() if b is not None]


def _find_experts(block: nn.Module):
    for name, sub in block.named_modules():
        if name.endswith("moe.experts") or name == "experts":
            return sub
    return None


def _odd_dtype_modules(block: nn.Module, skip: nn.Module | None = None) -> list[nn.Module]:
    """Submodules of `block` whose own parameters are stored in another dtype than most of the block (by element
    count).  Modules under `skip` (experts that already form a group) are left out."""
    skipped = {id(p) for p in skip.parameters()} if skip is not None else set()
    params = [p for p in block.parameters() if id(p) not in skipped]
    if not params:
        return []
    count: dict[torch.dtype, int] = {}
    for p in params:
        count[p.dtype] = count.get(p.dtype, 0) + p.numel()
    if len(count) == 1:
        return []
    major = max(count, key=count.get)
    odd = []
    for name, m in block.named_modules():
        own = [p for p in m.parameters(recurse=False) if id(p) not in skipped]
        if not own or all(p.dtype == major for p in own):
            continue
        if any(p.dtype == major for p in own):
            raise ValueError(f"module {name!r} mixes {major} parameters with others; FSDP needs one dtype per module")
        odd.append(m)
    return odd


def apply_fsdp(
    model: nn.Module,
    dp_mesh: DeviceMesh,
    *,
    param_dtype: torch.dtype = torch.bfloat16,
    reduce_dtype: torch.dtype = torch.float32,
    pp_enabled: bool = False,
    cpu_offload: bool = False,
    reshard_after_forward_policy: str = "default",
    ep_degree: int = 1,
    edp_mesh: DeviceMesh | None = None,
    gradient_divide_factor: int | None = None,
    layers_attr: str = "layers",
    extra_modules: tuple[str, ...] = (),
    ignored_params: set | None = None,
    reduce_scatter: str = "nccl",
    all_gather: str = "nccl",
) -> nn.Module:
    """Shard `model` block by block over `dp_mesh` (1-D = FSDP, 2-D = HSDP).  ``ignored_params``: parameters that
    another mechanism already shards (the fused-collective linears) and FSDP2 must leave alone.  ``reduce_scatter``:
    `nccl`, `peer_memory` or `auto` (see `titan_b200.parallel.fsdp_comm`)."""
    mp = MixedPrecisionPolicy(param_dtype=param_dtype, reduce_dtype=reduce_dtype)
    cfg = {"mesh": dp_mesh, "mp_policy": mp}
    if ignored_params:
        cfg["ignored_params"] = set(ignored_params)
    if cpu_offload:
        cfg["offload_policy"] = CPUOffloadPolicy()
    reshard = reshard_policy(reshard_after_forward_policy, pp_enabled)

    tok = getattr(model, "tok_embeddings", None)
    if tok is not None:
        fully_shard(tok, **cfg, reshard_after_forward=reshard)

    for _, block in _blocks(model, layers_attr):
        experts = _find_experts(block) if ep_degree > 1 else None
        if experts is not None:
            if edp_mesh is None:
                raise ValueError("edp_mesh is required when ep_degree > 1")
            ecfg = dict(cfg, mesh=edp_mesh)
            # shard experts on dim 1 when there are fewer local experts than efsdp ranks
            n_local = getattr(experts, "num_local_experts", None) or getattr(experts, "num_experts", 0) // ep_degree
            shard_fn = None
            if n_local and edp_mesh.size() > n_local:
                from torch.distributed.tensor import Shard

                shard_fn = lambda p: Shard(1)  # noqa: E731
            fully_shard(experts, **ecfg, reshard_after_forward=reshard, shard_placement_fn=shard_fn)
            if gradient_divide_factor is not None:
                experts.set_gradient_divide_factor(float(gradient_divide_factor))
        for odd in _odd_dtype_modules(block, skip=experts):
            # e.g. an fp32 gate inside a bf16-stored block: FSDP2 wants one storage dtype per group, so the module
            # becomes a group of its own that keeps its dtype in compute as well (library collectives: it is small)
            fully_shard(odd, **dict(cfg, mp_policy=MixedPrecisionPolicy(param_dtype=None, reduce_dtype=reduce_dtype)),
                        reshard_after_forward=reshard)
            odd._keeps_library_collectives = True
            if gradient_divide_factor is not None and experts is not None:
                odd.set_gradient_divide_factor(float(gradient_divide_factor))
        fully_shard(block, **cfg, reshard_after_forward=reshard)
        if gradient_divide_factor is not None and experts is not None:
            block.set_gradient_divide_factor(float(gradient_divide_factor))

    for name in extra_modules:
        sub = model.get_submodule(name) if name else None
        if sub is not None:
            fully_shard(sub, **cfg, reshard_after_forward=reshard)

    norm, output = getattr(model, "norm", None), getattr(model, "output", None)
    tail = [m for m in (norm, output) if m is not None]
    if tail:
        # the last group is never resharded after forward: backward needs it immediately
        fully_shard(tail, **cfg, reshard_after_forward=reshard_after_forward_policy == "always")
    fully_shard(model, **cfg, reshard_after_forward=reshard)
    if gradient_divide_factor is not None and ep_degree > 1:
        model.set_gradient_divide_factor(float(gradient_divide_factor))
    if not cpu_offload:
        from titan_b200.parallel.fsdp_comm import install_peer_reduce_scatter, peer_reduce_scatter_wanted

        from titan_b200.parallel.fsdp_comm import install_peer_all_gather

        if peer_reduce_scatter_wanted(reduce_scatter, dp_mesh, dp_mesh.device_type):
            model._peer_reduce_scatter = install_peer_reduce_scatter(model, dp_mesh, wire_dtype=param_dtype,
                                                                     nvls=reduce_scatter == "nvls")
        if peer_reduce_scatter_wanted(all_gather, dp_mesh, dp_mesh.device_type):
            model._peer_all_gather = install_peer_all_gather(model, dp_mesh, param_dtype=param_dtype)
    return model


def apply_replicate(model: nn.Module, dp_mesh: DeviceMesh, *, param_dtype=torch.bfloat16,
                    reduce_dtype=torch.float32, layers_attr: str = "layers") -> nn.Module:
    """Pure data parallel expressed as FSDP2 that never reshards (replicate-with-FSDP).

    ``dp_mesh`` is the 2-D ``(dp_replicate, fsdp)`` mesh with a trivial shard axis, sliced from a mesh that covers
    the whole job (`ParallelDims.get_mesh(("dp_replicate", "fsdp"))`): every rank then creates the same process
    groups in the same order.  A 1-D mesh is accepted only when it spans the whole job, where building the 2-D
    layout locally is equally collective; with tp / pp / cp ranks alongside, per-rank sub-meshes would call
    `new_group` with rank lists that differ between ranks."""
    mp = MixedPrecisionPolicy(param_dtype=param_dtype, reduce_dtype=reduce_dtype)
    if dp_mesh.ndim == 1:
        import torch.distributed as dist

        if dist.is_initialized() and dp_mesh.size() != dist.get_world_size():
            raise ValueError("apply_replicate needs the 2-D (dp_replicate, fsdp) mesh when other parallel axes exist")
        ranks = dp_mesh.mesh.view(-1, 1)
        dp_mesh = DeviceMesh(dp_mesh.device_type, ranks, mesh_dim_names=("dp_replicate", "dp_shard_1"))
    for _, block in _blocks(model, layers_attr):
        fully_shard(block, mesh=dp_mesh, mp_policy=mp, reshard_after_forward=False)
    fully_shard(model, mesh=dp_mesh, mp_policy=mp, reshard_after_forward=False)
    return model
