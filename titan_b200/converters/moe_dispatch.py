"""`b200_moe_dispatch` (alias `npu_moe_dispatch`): `MoE` → `FusedMoE`.

The fused layer routes with the router-top-k kernel, builds a routing plan on the device (no host
sync for split sizes), permutes straight into the padded expert-major layout, runs the experts and
combines with the weighted un-permute kernel (+ shared-expert output in the same pass).  Under expert
parallelism the plan updater swaps the NCCL `ExpertParallel` style for `FusedExpertParallel`, whose
dispatch / combine kernels write and read peers' buffers over NVLink.

Parity: torchtitan_npu/converters/kernels/moe_dispatch.py:74-287 (NpuMoE, NpuExpertParallel plan swap).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from titan_b200.converters.convert_utils import replace_modules
from titan_b200.models.common.moe import MoE
from titan_b200.ops import moe as moe_ops
from titan_b200.parallel.expert_parallel import ExpertParallel, FusedExpertParallel
from titan_b200.protocols.converter import ConverterSpec, ModelConverter, PlanUpdater, register_model_converter

__all__ = ["FusedMoE", "ExpertParallelPlanUpdater"]


class FusedMoE(MoE):
    def forward(self, x: torch.Tensor, input_ids: torch.Tensor | None = None) -> torch.Tensor:
        experts = self.experts
        if not hasattr(experts, "forward_padded"):
            return super().forward(x, input_ids)  # experts not converted: nothing to fuse against
        bs, slen, dim = x.shape
        x2 = x.reshape(-1, dim)
        T = x2.shape[0]
        r = self.router
        logits = F.linear(x2.float(), r.gate_weight().float())
        forced = None
        if r.hash:
            forced = r.tid2eid[input_ids.flatten()]
        elif r._debug_force_load_balance:
            forced = (torch.arange(T * r.top_k, device=x.device).view(T, r.top_k)) % r.num_experts
        if r.num_expert_groups and r.num_limited_groups and forced is None:
            # group-limited choice is a masking step on the [T, E] matrix: done in PyTorch, gate values by kernel
            scores = r._scores(logits)
            choice = scores if self.expert_bias is None else scores + self.expert_bias
            forced = r._group_limited(choice).topk(r.top_k, dim=-1)[1]
        gate, idx, counts = moe_ops.router_topk(logits, r.top_k, bias=self.expert_bias, score_func=r.score_func,
                                                route_norm=r.route_norm, route_scale=r.route_scale,
                                                forced_idx=forced)
        with torch.no_grad():
            self.tokens_per_expert.add_(counts.to(self.tokens_per_expert.dtype))
        base = self.shared_experts(x2) if self.shared_experts is not None else None
        ep_mesh = getattr(experts, "ep_mesh", None)
        if ep_mesh is not None and ep_mesh.size() > 1:
            if not x.is_cuda:
                raise RuntimeError("the fused expert-parallel MoE exchanges tokens through GPU peer memory; on CPU run "
                                   "expert parallelism without the b200_moe_dispatch / b200_gmm converters")
            from titan_b200.ops import moe_comm

            out = moe_comm.moe_forward_ep(x2, gate, idx, experts, ep_mesh.get_group(), base=base,
                                          score_before_experts=self.score_before_experts)
            return out.reshape(bs, slen, dim)
        plan = moe_ops.make_plan(idx, r.num_experts)
        if self.score_before_experts:
            xp = moe_ops.permute(x2, plan, scale=gate)
            yp = experts(xp, plan.offs, padded=True)
            out = moe_ops.combine(yp, plan, T, weights=None, base=base)
        else:
            xp = moe_ops.permute(x2, plan)
            yp = experts(xp, plan.offs, padded=True)
            out = moe_ops.combine(yp, plan, T, weights=self.full_grad(gate), base=base)
        return out.reshape(bs, slen, dim)


def _swap(old: MoE) -> FusedMoE:
    new = FusedMoE.__new__(FusedMoE)
    new.__dict__ = old.__dict__
    return new


class MoEDispatchConverter(ModelConverter):
    def convert(self, model) -> None:
        self.replaced = replace_modules(model, r"MoE", _swap)


class ExpertParallelPlanUpdater(PlanUpdater):
    @classmethod
    def update(cls, plan):
        if type(plan) is ExpertParallel:
            return FusedExpertParallel()
        if isinstance(plan, dict):
            return {k: (FusedExpertParallel() if type(v) is ExpertParallel else v) for k, v in plan.items()}
        return plan


MOE_DISPATCH = register_model_converter("b200_moe_dispatch", "npu_moe_dispatch")(
    ConverterSpec(model_converter=MoEDispatchConverter, plan_updater=ExpertParallelPlanUpdater))
