"""`b200_gmm` (alias `npu_gmm`): `GroupedExperts` → `FusedGroupedExperts`.

``w1`` and ``w3`` are fused into ``w13 [E, 2H, D]`` (rows ``[w1 | w3]``) so the up-projection is one
grouped GEMM; the activation is the fused clamp + SwiGLU (+ routed score) kernel; both grouped GEMMs
run on the tcgen05 grouped kernel over the padded expert-major layout.  `GMMStateDictUpdater` keeps
checkpoints in the canonical ``w1 / w3`` layout (split on export, fuse on import, drop
``.weight_scale_inv`` entries of quantised checkpoints).

Parity: torchtitan_npu/converters/kernels/gmm.py:87-331.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from titan_b200.checkpoint.weight_utils import fuse_experts, split_fused_experts
from titan_b200.converters.convert_utils import replace_modules
from titan_b200.models.common.moe import GroupedExperts
from titan_b200.ops.moe import grouped_linear
from titan_b200.ops.swiglu import swiglu_fused
from titan_b200.protocols.converter import (
    ConverterSpec,
    ModelConverter,
    StateDictUpdater,
    register_model_converter,
)
from titan_b200.protocols.module import Module

__all__ = ["FusedGroupedExperts", "GMMStateDictUpdater"]


class FusedGroupedExperts(Module):
    def __init__(self, dim: int, hidden_dim: int, num_experts: int, swiglu_limit: float = 0.0, device=None,
                 dtype=None):
        super().__init__()
        self.num_experts, self.hidden_dim, self.dim = num_experts, hidden_dim, dim
        self.w13 = nn.Parameter(torch.empty(num_experts, 2 * hidden_dim, dim, device=device, dtype=dtype))
        self.w2 = nn.Parameter(torch.empty(num_experts, dim, hidden_dim, device=device, dtype=dtype))
        self.swiglu_limit = swiglu_limit
        self.use_grouped_mm = True

    @staticmethod
    def _local(p):
        return p.to_local() if hasattr(p, "to_local") else p

    def _weights_resident(self) -> bool:
        """False when FSDP shards this module's weights over more than one rank: the gathered copy is transient there,
        and a cache of its quantised views would pin the unsharded bytes."""
        if not hasattr(self, "_get_fsdp_state"):
            return True
        try:
            group = self._get_fsdp_state()._fsdp_param_group
            return group is None or group.mesh_info.shard_mesh_size <= 1
        except Exception:  # noqa: BLE001
            return False

    def forward_padded(self, xp: torch.Tensor, offs: torch.Tensor, scores: torch.Tensor | None = None):
        """xp: padded expert-major rows [cap, D]; offs: cumulative padded ends of the LOCAL experts."""
        w13, w2 = self._local(self.w13), self._local(self.w2)
        mx = getattr(self, "mx_round_mode", None)
        if mx is not None:  # MXFP8 experts: both GEMMs block-quantised along their contraction dims
            # a weight that stays whole on this rank keeps its quantised views between optimizer steps
            k13, k2 = ((id(self), "w13"), (id(self), "w2")) if self._weights_resident() else (None, None)
            kw = {"weight_key": k13} if k13 is not None else {}
            h13 = self.mx_grouped_mm(xp, w13.to(xp.dtype), offs, mx, aligned=True, **kw)  # groups: 128-row multiples
            h = swiglu_fused(h13, scores, self.swiglu_limit)
            kw = {"weight_key": k2} if k2 is not None else {}
            return self.mx_grouped_mm(h, w2.to(xp.dtype), offs, mx, aligned=True, **kw)
        h13 = grouped_linear(xp, w13.to(xp.dtype), offs)
        h = swiglu_fused(h13, scores, self.swiglu_limit)
        return grouped_linear(h, w2.to(xp.dtype), offs)

    def forward(self, x: torch.Tensor, num_tokens_per_expert: torch.Tensor, scores: torch.Tensor | None = None,
                padded: bool = False) -> torch.Tensor:
        """Unpadded expert-sorted rows (the layout of the NCCL expert-parallel path); ``padded=True`` takes the
        128-row-padded layout with cumulative ends instead.  The fused MoE layer calls the module (not
        `forward_padded` directly) so that FSDP's unshard / gradient-reduction hooks run around the experts."""
        if padded:
            return self.forward_padded(x, num_tokens_per_expert, scores)
        w13, w2 = self._local(self.w13), self._local(self.w2)
        offs = torch.cumsum(num_tokens_per_expert, 0, dtype=torch.int32)
        mx = getattr(self, "mx_round_mode", None)
        if mx is not None:
            h13 = self.mx_grouped_mm(x, w13.to(x.dtype), offs, mx)
            return self.mx_grouped_mm(swiglu_fused(h13, None, self.swiglu_limit), w2.to(x.dtype), offs, mx)
        if x.is_cuda or x.is_meta:
            h13 = torch._grouped_mm(x.bfloat16(), w13.bfloat16().transpose(-2, -1), offs=offs)
            h = swiglu_fused(h13, None, self.swiglu_limit)
            return torch._grouped_mm(h, w2.bfloat16().transpose(-2, -1), offs=offs).to(x.dtype)
        outs, start = [], 0
        for e, end in enumerate(offs.tolist()):
            h13 = x[start:end] @ w13[e].t()
            outs.append(swiglu_fused(h13, None, self.swiglu_limit) @ w2[e].t())
            start = end
        if start < x.shape[0]:
            outs.append(x.new_zeros(x.shape[0] - start, w2.shape[1]))
        return torch.cat(outs, dim=0)

    def init_states(self, *, init_std: float = 0.02, **kw):
        h = self.hidden_dim
        with torch.no_grad():
            w13 = self._local(self.w13)
            nn.init.trunc_normal_(w13[:, :h], mean=0.0, std=0.02)
            nn.init.trunc_normal_(w13[:, h:], mean=0.0, std=init_std)
        nn.init.trunc_normal_(self.w2, mean=0.0, std=init_std)


def _swap(old: GroupedExperts) -> FusedGroupedExperts:
    e, h, d = old.w1.shape
    return FusedGroupedExperts(d, h, e, old.swiglu_limit, device=old.w1.device, dtype=old.w1.dtype)


class GMMConverter(ModelConverter):
    def convert(self, model) -> None:
        self.replaced = replace_modules(model, r"GroupedExperts", _swap)


class GMMStateDictUpdater(StateDictUpdater):
    @classmethod
    def to_hf(cls, state_dict):
        return split_fused_experts(dict(state_dict))

    @classmethod
    def from_hf(cls, state_dict):
        sd = {k: v for k, v in state_dict.items() if not k.endswith(".weight_scale_inv")}
        return fuse_experts(sd)


GMM = register_model_converter("b200_gmm", "npu_gmm")(
    ConverterSpec(model_converter=GMMConverter, state_dict_updater=GMMStateDictUpdater))
