"""Context parallelism for DeepSeek sparse attention (DSA): all-gather the shared KV latent and indexer keys.

Queries stay sequence-local.  The single-head KV latent ``k, v [B, 1, S/cp, D]`` and the indexer keys
``k_indexer [B, S/cp, 1, 128]`` are all-gathered over the ``cp`` mesh (small: one head), then cut to the
causal prefix ``[: (rank + 1) · S_local]`` so rank r attends to everything up to its own block; the
attention core treats the local queries as the tail of that key range.  Backward of the gather is a
reduce-scatter (functional collective with autograd).  Work grows with the rank; no balancing is applied
because top-k selection bounds the attention cost and the indexer is cheap.

Parity: torchtitan_npu/distributed/context_parallel/sparse_attention_cp.py:30-90.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch.distributed._functional_collectives import all_gather_tensor_autograd
from torch.distributed.device_mesh import DeviceMesh

from titan_b200.parallel.context_parallel.registry import register_cp_strategy
from titan_b200.parallel.fake_pg import is_fake_process_group

__all__ = ["SparseAttentionCP"]


def _gather(x: torch.Tensor, dim: int, group, world: int) -> torch.Tensor:
    if world == 1:
        return x
    if is_fake_process_group(group):
        return torch.cat([x] * world, dim=dim)
    out = all_gather_tensor_autograd(x.contiguous(), gather_dim=dim, group=group)
    # wait on the functional tensor (not `.wait()` of the async wrapper) so autograd keeps the edge
    return torch.ops._c10d_functional.wait_tensor(out)


class SparseAttentionCP:
    def __init__(self, cp_mesh: DeviceMesh):
        self.group = cp_mesh.get_group()
        self.cp, self.rank = cp_mesh.size(), cp_mesh.get_local_rank()

    def pre(self, module, args, kwargs):
        q, k, v, *rest = args
        s_local = k.shape[2]
        keep = (self.rank + 1) * s_local
        k = _gather(k, 2, self.group, self.cp)[:, :, :keep]
        v = _gather(v, 2, self.group, self.cp)[:, :, :keep]
        kw = dict(kwargs)
        if kw.get("k_indexer") is not None:
            kw["k_indexer"] = _gather(kw["k_indexer"], 1, self.group, self.cp)[:, :keep]
        if kw.get("attn_mask") is not None:
            raise NotImplementedError("DSA CP builds its own causal mask; custom masks are not supported")
        return (q, k, v, *rest), kw

    def apply(self, module: nn.Module) -> nn.Module:
        module.register_forward_pre_hook(self.pre, with_kwargs=True)
        module._cp_strategy = "dsa_allgather"
        return module


def _is_dsa_core(mod: nn.Module) -> bool:
    return getattr(mod, "cp_layout", None) == "dsa" or type(mod).__name__ in ("DSASparseAttention", "FusedDSAttention")


register_cp_strategy("dsa_allgather", _is_dsa_core, lambda m, mesh: SparseAttentionCP(mesh).apply(m), first=True)
