"""Mixture-of-experts building blocks (baseline PyTorch math).

`TokenChoiceTopKRouter` → `TokenReorderer` → `GroupedExperts` → weighted scatter-add, plus shared
experts and the auxiliary-loss-free load-balancing buffers (`expert_bias`, `tokens_per_expert`).
Expert weights are stacked ``w1, w3: [E, H, D]``, ``w2: [E, D, H]`` so one grouped GEMM serves all
local experts.  The fused sm_100a paths (router top-k, permute, grouped GEMM, SwiGLU with score,
peer-memory dispatch/combine) replace pieces of this module through converters.

Parity: upstream `MoE / TokenChoiceTopKRouter / TokenReorderer / GroupedExperts` as used and
extended by the reference (torchtitan_npu/models/deepseek_v4/moe.py:21-413: sqrt-softplus scores,
hash routing table, SwiGLU clamp, forced load balance; converters/kernels/moe_dispatch.py:74-107).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from titan_b200.models.common.layers import FeedForward, Linear
from titan_b200.protocols.module import Module

__all__ = ["MoEArgs", "TokenChoiceTopKRouter", "TokenReorderer", "GroupedExperts", "MoE", "build_hash_routing_table",
           "run_experts_for_loop", "run_experts_grouped_mm", "softplus_stable"]


@dataclass
class MoEArgs:
    num_experts: int = 8
    num_shared_experts: int = 1
    top_k: int = 1
    score_func: str = "sigmoid"  # sigmoid | softmax | sqrtsoftplus
    route_norm: bool = False
    route_scale: float = 1.0
    score_before_experts: bool = True
    use_grouped_mm: bool = True
    load_balance_coeff: float | None = 1e-3
    num_expert_groups: int | None = None
    num_limited_groups: int | None = None
    swiglu_limit: float = 0.0
    n_hash_layers: int = 0
    _debug_force_load_balance: bool = False


def softplus_stable(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 20, x, torch.log1p(torch.exp(torch.clamp(x, max=20))))


def build_hash_routing_table(vocab_size: int, num_experts: int, top_k: int, device=None, seed: int = 0):
    """Fixed token-id → expert-ids table ``[vocab, top_k]`` (distinct experts per token, deterministic)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    base = torch.randint(0, num_experts, (vocab_size, 1), generator=g, device="cpu")
    step = max(num_experts // max(top_k, 1), 1)
    table = (base + torch.arange(top_k, device="cpu").view(1, -1) * step) % num_experts
    return table.to(device=device, dtype=torch.int64)


class TokenChoiceTopKRouter(Module):
    def __init__(self, dim: int, args: MoEArgs, *, layer_id: int = 0, vocab_size: int = 0):
        super().__init__()
        self.gate = Linear(dim, args.num_experts, bias=False)
        self.num_experts, self.top_k = args.num_experts, args.top_k
        self.score_func, self.route_norm, self.route_scale = args.score_func, args.route_norm, args.route_scale
        self.num_expert_groups, self.num_limited_groups = args.num_expert_groups, args.num_limited_groups
        self._debug_force_load_balance = args._debug_force_load_balance
        self.hash = layer_id < args.n_hash_layers
        self.vocab_size = vocab_size
        if self.hash:
            self.register_buffer("tid2eid", build_hash_routing_table(vocab_size, self.num_experts, self.top_k),
                                 persistent=True)

    def gate_weight(self) -> torch.Tensor:
        """Local gate weight.  Under tensor parallelism it is replicated; when every rank routes only its own
        sequence slice (``tokens_sharded``) the gradient is a partial sum and is reduced over the mesh."""
        from titan_b200.parallel.tensor_parallel import replicated_param_local

        return replicated_param_local(self.gate.weight, partial_grad=getattr(self, "tokens_sharded", False))

    def _scores(self, logits: torch.Tensor) -> torch.Tensor:
        if self.score_func == "sigmoid":
            return torch.sigmoid(logits)
        if self.score_func == "softmax":
            return F.softmax(logits, dim=1)
        if self.score_func == "sqrtsoftplus":
            return softplus_stable(logits).sqrt()
        raise NotImplementedError(f"unknown score function {self.score_func}")

    def _force_balanced(self, scores: torch.Tensor):
        n = scores.shape[0]
        idx = (torch.arange(n * self.top_k, device=scores.device).view(n, self.top_k)) % self.num_experts
        return idx, scores.gather(1, idx)

    def _group_limited(self, scores_for_choice: torch.Tensor) -> torch.Tensor:
        n = scores_for_choice.shape[0]
        g = self.num_expert_groups
        grouped = scores_for_choice.view(n, g, -1)
        group_scores = grouped.topk(2, dim=-1)[0].sum(-1) if grouped.shape[-1] >= 2 else grouped.amax(-1)
        keep = group_scores.topk(self.num_limited_groups, dim=-1)[1]
        mask = torch.ones(n, g, dtype=torch.bool, device=scores_for_choice.device).scatter_(1, keep, False)
        return grouped.masked_fill(mask.unsqueeze(-1), float("-inf")).view(n, -1)

    def forward(self, x: torch.Tensor, expert_bias: torch.Tensor | None = None, input_ids: torch.Tensor | None = None):
        """x [T, dim] → (top_scores [T, k] fp32, selected [T, k] int64, tokens_per_expert [E] fp32)."""
        logits = F.linear(x.float(), self.gate_weight().float())  # routing in fp32
        scores = self._scores(logits)
        if self.hash:
            if input_ids is None:
                raise ValueError("hash routing needs input_ids")
            selected = self.tid2eid[input_ids.flatten()]
        else:
            choice = scores if expert_bias is None else scores + expert_bias
            if self.num_expert_groups and self.num_limited_groups:
                choice = self._group_limited(choice)
            selected = choice.topk(self.top_k, dim=-1)[1]
        top_scores = scores.gather(1, selected)  # the bias steers the choice only, not the gate value
        if self._debug_force_load_balance:
            selected, top_scores = self._force_balanced(scores)
        if self.route_norm:
            top_scores = top_scores / (top_scores.sum(-1, keepdim=True) + 1e-20)
        top_scores = top_scores * self.route_scale
        # integer counts: FSDP's mixed-precision policy casts floating-point forward inputs of the experts module to
        # bf16, which cannot hold counts above 256 exactly (the all-to-all split sizes would no longer add up)
        counts = torch.histc(selected.reshape(-1).float(), bins=self.num_experts, min=0,
                             max=self.num_experts).to(torch.int64)
        return top_scores, selected, counts

    def init_states(self, *, init_std: float = 0.02, **kw):
        nn.init.trunc_normal_(self.gate.weight, mean=0.0, std=init_std)
        if self.hash:
            self.tid2eid = build_hash_routing_table(self.vocab_size, self.num_experts, self.top_k,
                                                    device=self.gate.weight.device)


class TokenReorderer(Module):
    """Sort the T·k (token, expert) pairs by expert id (stable) so each expert's tokens are contiguous."""

    def __init__(self, num_experts: int, top_k: int):
        super().__init__()
        self.num_experts, self.top_k = num_experts, top_k

    def forward(self, top_scores: torch.Tensor, selected: torch.Tensor):
        order = torch.argsort(selected.reshape(-1), stable=True)
        scores_sorted = top_scores.reshape(-1)[order]
        token_idx_sorted = order // self.top_k
        return scores_sorted, token_idx_sorted, order


def run_experts_for_loop(w1, w2, w3, x, counts, limit: float = 0.0):
    outs = []
    splits = counts.tolist() if isinstance(counts, torch.Tensor) else list(counts)
    splits = [int(s) for s in splits]
    pad = x.shape[0] - sum(splits)
    chunks = torch.split(x[: sum(splits)], splits, dim=0)
    for e, xe in enumerate(chunks):
        g, u = xe @ w1[e].t(), xe @ w3[e].t()
        if limit > 0:
            g, u = g.clamp(max=limit), u.clamp(min=-limit, max=limit)
        outs.append((F.silu(g) * u) @ w2[e].t())
    out = torch.cat(outs, dim=0) if outs else x.new_zeros(0, w2.shape[1])
    if pad > 0:
        out = torch.cat([out, out.new_zeros(pad, out.shape[-1])], dim=0)
    return out


def run_experts_grouped_mm(w1, w2, w3, x, counts, limit: float = 0.0):
    offs = torch.cumsum(counts, dim=0, dtype=torch.int32)
    dt = x.dtype
    xb = x.bfloat16()
    g = torch._grouped_mm(xb, w1.bfloat16().transpose(-2, -1), offs=offs)
    u = torch._grouped_mm(xb, w3.bfloat16().transpose(-2, -1), offs=offs)
    if limit > 0:
        g, u = g.clamp(max=limit), u.clamp(min=-limit, max=limit)
    h = F.silu(g) * u
    return torch._grouped_mm(h, w2.bfloat16().transpose(-2, -1), offs=offs).to(dt)


class GroupedExperts(Module):
    def __init__(self, dim: int, hidden_dim: int, num_experts: int, use_grouped_mm: bool = True,
                 swiglu_limit: float = 0.0):
        super().__init__()
        self.num_experts = num_experts
        self.w1 = nn.Parameter(torch.empty(num_experts, hidden_dim, dim))
        self.w2 = nn.Parameter(torch.empty(num_experts, dim, hidden_dim))
        self.w3 = nn.Parameter(torch.empty(num_experts, hidden_dim, dim))
        self.use_grouped_mm = use_grouped_mm
        self.swiglu_limit = swiglu_limit

    def _local(self, p):
        return p.to_local() if hasattr(p, "to_local") else p

    def forward(self, x: torch.Tensor, num_tokens_per_expert: torch.Tensor) -> torch.Tensor:
        w1, w2, w3 = self._local(self.w1), self._local(self.w2), self._local(self.w3)
        counts = num_tokens_per_expert
        mx = getattr(self, "mx_round_mode", None)
        if mx is not None:  # MXFP8 experts (set by the MXFP8 converter)
            offs = torch.cumsum(counts, 0, dtype=torch.int32)
            g, u = self.mx_grouped_mm(x, w1.to(x.dtype), offs, mx), self.mx_grouped_mm(x, w3.to(x.dtype), offs, mx)
            if self.swiglu_limit > 0:
                g, u = g.clamp(max=self.swiglu_limit), u.clamp(min=-self.swiglu_limit, max=self.swiglu_limit)
            return self.mx_grouped_mm(F.silu(g) * u, w2.to(x.dtype), offs, mx)
        if (self.use_grouped_mm and x.is_cuda) or x.is_meta:   # meta: shapes only (no host read of the counts)
            return run_experts_grouped_mm(w1, w2, w3, x, counts.to(torch.int32), self.swiglu_limit)
        return run_experts_for_loop(w1, w2, w3, x, counts.long(), self.swiglu_limit)

    def init_states(self, *, init_std: float = 0.02, **kw):
        nn.init.trunc_normal_(self.w1, mean=0.0, std=0.02)
        nn.init.trunc_normal_(self.w2, mean=0.0, std=init_std)
        nn.init.trunc_normal_(self.w3, mean=0.0, std=init_std)


class MoE(Module):
    def __init__(self, dim: int, hidden_dim: int, args: MoEArgs, *, layer_id: int = 0, vocab_size: int = 0):
        super().__init__()
        self.args = args
        self.experts = GroupedExperts(dim, hidden_dim, args.num_experts, args.use_grouped_mm, args.swiglu_limit)
        self.router = TokenChoiceTopKRouter(dim, args, layer_id=layer_id, vocab_size=vocab_size)
        self.reorderer = TokenReorderer(args.num_experts, args.top_k)
        self.shared_experts = (FeedForward(dim=dim, hidden_dim=hidden_dim * args.num_shared_experts)
                               if args.num_shared_experts > 0 else None)
        self.score_before_experts = args.score_before_experts
        self.load_balance_coeff = args.load_balance_coeff
        if self.load_balance_coeff is not None:
            self.register_buffer("expert_bias", torch.zeros(args.num_experts, dtype=torch.float32), persistent=True)
        else:
            self.expert_bias = None
        self.register_buffer("tokens_per_expert", torch.zeros(args.num_experts, dtype=torch.float32),
                             persistent=False)

    def full_grad(self, gate_values: torch.Tensor) -> torch.Tensor:
        """Gate values that multiply a routed output which is a PARTIAL sum over tensor-parallel ranks receive a
        partial gradient; it is summed over ``tp_partial_group`` (set by the parallelize plan) in backward."""
        group = getattr(self, "tp_partial_group", None)
        if group is None or not gate_values.requires_grad:
            return gate_values
        from titan_b200.parallel.expert_parallel import _AllReduceGrad

        return _AllReduceGrad.apply(gate_values, group)

    def forward(self, x: torch.Tensor, input_ids: torch.Tensor | None = None) -> torch.Tensor:
        bs, slen, dim = x.shape
        x2 = x.reshape(-1, dim)
        top_scores, selected, counts = self.router(x2, self.expert_bias, input_ids)
        with torch.no_grad():
            self.tokens_per_expert.add_(counts)
        scores_sorted, token_idx, _ = self.reorderer(top_scores, selected)
        routed_in = x2[token_idx]
        if self.score_before_experts:
            routed_in = (routed_in.float() * scores_sorted.reshape(-1, 1)).to(x.dtype)
        routed_out = self.experts(routed_in, counts)
        if not self.score_before_experts:
            routed_out = (routed_out.float() * self.full_grad(scores_sorted).reshape(-1, 1)).to(x.dtype)
        out = self.shared_experts(x2) if self.shared_experts is not None else torch.zeros_like(x2)
        out = out.index_add(0, token_idx, routed_out.to(out.dtype))
        return out.reshape(bs, slen, dim)

    def init_states(self, *, init_std: float = 0.02, buffer_device=None, **kw):
        self.experts.init_states(init_std=init_std)
        self.router.init_states(init_std=init_std)
        if self.shared_experts is not None:
            self.shared_experts.init_states(init_std=init_std)
        dev = buffer_device or self.tokens_per_expert.device
        with torch.device(dev):
            self.tokens_per_expert = torch.zeros(self.args.num_experts, dtype=torch.float32)
            if self.load_balance_coeff is not None:
                self.expert_bias = torch.zeros(self.args.num_experts, dtype=torch.float32)
