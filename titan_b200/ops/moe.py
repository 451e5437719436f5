"""MoE operators on sm_100a kernels: router top-k, padded expert-major permutation, grouped GEMM.

Data flow of one MoE layer on the fused path (no host synchronisation anywhere):

    logits ─ router_topk ─► gate [T,k], idx [T,k], counts [E]
    idx ─ plan ─► dest [T·k] (row of every (token, slot) pair), offs [E] (padded cumulative ends)
    x ─ permute(dest) ─► xp [cap, D]      (expert-major, every expert padded to 128 rows, pads zero)
    xp ─ grouped_linear(w13, offs) ─ swiglu(+gate) ─ grouped_linear(w2, offs) ─► yp [cap, D]
    yp ─ combine(dest, gate) (+ shared-expert output) ─► y [T, D]

`cap = T·k + 127·E` bounds the padded row count, so buffers are sized without knowing the routing.
Every function has a PyTorch oracle (`*_ref`) used for CPU execution and for tests.

Parity: K4/K5/K6/K24 of the reference op library (ops/_grouped_mm.py:10-42,
converters/kernels/permutation.py:13-143, models/deepseek_v4/moe.py:125-187).
"""

from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from titan_b200.ops import _lib

__all__ = ["router_topk", "router_topk_ref", "MoePlan", "make_plan", "permute", "combine", "grouped_linear",
           "grouped_linear_ref", "capacity_for", "ALIGN"]

ALIGN = 128
_SCORE = {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}


def _on_device(t: torch.Tensor) -> bool:
    """CUDA tensors run the kernels; meta tensors follow the same path with the launches skipped, so shapes, saved
    tensors and buffer sizes are those of a GPU run (the memory simulator relies on it)."""
    return t.is_cuda or t.is_meta


def capacity_for(num_pairs: int, num_experts: int) -> int:
    return (num_pairs + (ALIGN - 1) * num_experts + ALIGN - 1) // ALIGN * ALIGN


# ------------------------------------------------------------------------------ router
def _scores_torch(logits, score_func):
    if score_func == "sigmoid":
        return torch.sigmoid(logits)
    if score_func == "softmax":
        return F.softmax(logits, dim=-1)
    if score_func == "sqrtsoftplus":
        return torch.where(logits > 20, logits, torch.log1p(torch.exp(torch.clamp(logits, max=20)))).sqrt()
    raise NotImplementedError(score_func)


def router_topk_ref(logits, k, *, bias=None, score_func="sigmoid", route_norm=False, route_scale=1.0,
                    forced_idx=None):
    scores = _scores_torch(logits.float(), score_func)
    if forced_idx is None:
        choice = scores if bias is None else scores + bias
        idx = choice.topk(k, dim=-1)[1]
    else:
        idx = forced_idx
    gate = scores.gather(1, idx)
    if route_norm:
        gate = gate / (gate.sum(-1, keepdim=True) + 1e-20)
    gate = gate * route_scale
    counts = torch.bincount(idx.reshape(-1), minlength=logits.shape[1]).to(torch.int32)
    return gate, idx, counts


class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, forced_idx, k, score_func, route_norm, route_scale):
        T, E = logits.shape
        logits = logits.float().contiguous()
        gate = torch.empty(T, k, dtype=torch.float32, device=logits.device)
        idx = torch.empty(T, k, dtype=torch.int64, device=logits.device)
        counts = torch.zeros(E, dtype=torch.int32, device=logits.device)
        rc = 0 if logits.is_meta else _lib.lib().tb_router_topk(
            logits.data_ptr(), _lib.ptr(bias.float().contiguous() if bias is not None else None),
            _lib.ptr(forced_idx.contiguous() if forced_idx is not None else None), gate.data_ptr(), idx.data_ptr(),
            counts.data_ptr(), None, T, E, k, _SCORE[score_func], int(route_norm), float(route_scale),
            _lib.shared_status().ptr, _lib.stream_ptr())
        _lib.check(rc, "router_topk")
        ctx.save_for_backward(logits, idx)
        ctx.cfg = (score_func, route_norm, route_scale)
        ctx.mark_non_differentiable(idx, counts)
        return gate, idx, counts

    @staticmethod
    def backward(ctx, g_gate, _gi, _gc):
        logits, idx = ctx.saved_tensors
        score_func, route_norm, route_scale = ctx.cfg
        # the [T, E] score matrix is tiny next to the expert GEMMs: differentiate it with PyTorch
        with torch.enable_grad():
            l = logits.detach().requires_grad_()
            gate = _scores_torch(l, score_func).gather(1, idx)
            if route_norm:
                gate = gate / (gate.sum(-1, keepdim=True) + 1e-20)
            gate = gate * route_scale
            (dl,) = torch.autograd.grad(gate, l, g_gate)
        return dl, None, None, None, None, None, None


def router_topk(logits, k, *, bias=None, score_func="sigmoid", route_norm=False, route_scale=1.0, forced_idx=None):
    """→ (gate [T,k] fp32, idx [T,k] int64, counts [E] int32)."""
    if not _on_device(logits):
        return router_topk_ref(logits, k, bias=bias, score_func=score_func, route_norm=route_norm,
                               route_scale=route_scale, forced_idx=forced_idx)
    return _RouterFn.apply(logits, bias, forced_idx, k, score_func, route_norm, route_scale)


# ------------------------------------------------------------------------------ plan / permute / combine
class MoePlan:
    """Routing plan of one layer: destination row per pair and padded expert offsets (all on device)."""

    def __init__(self, dest, counts, starts, offs, capacity, num_experts, top_k):
        self.dest, self.counts, self.starts, self.offs = dest, counts, starts, offs
        self.capacity, self.num_experts, self.top_k = capacity, num_experts, top_k


def _plan_ref(idx, E, capacity):
    flat = idx.reshape(-1)
    counts = torch.bincount(flat, minlength=E)
    padded = (counts + ALIGN - 1) // ALIGN * ALIGN
    offs = torch.cumsum(padded, 0)
    starts = offs - padded
    order = torch.argsort(flat, stable=True)
    rank_in_e = torch.empty_like(flat)
    seg_start = torch.cumsum(counts, 0) - counts
    rank_in_e[order] = torch.arange(flat.numel(), device=flat.device) - seg_start[flat[order]]
    dest = (starts[flat] + rank_in_e).to(torch.int32)
    return dest, counts.to(torch.int32), starts.to(torch.int32), offs.to(torch.int32)


def make_plan(idx: torch.Tensor, num_experts: int, capacity: int | None = None) -> MoePlan:
    T, k = idx.shape
    P = T * k
    capacity = capacity or capacity_for(P, num_experts)
    if not _on_device(idx):
        dest, counts, starts, offs = _plan_ref(idx, num_experts, capacity)
        return MoePlan(dest, counts, starts, offs, capacity, num_experts, k)
    dev = idx.device
    if idx.is_meta:
        dest = torch.empty(P, dtype=torch.int32, device=dev)
        counts, starts, offs = (torch.empty(num_experts, dtype=torch.int32, device=dev) for _ in range(3))
        return MoePlan(dest, counts, starts, offs, capacity, num_experts, k)
    L = _lib.lib()
    nb = L.tb_moe_plan_blocks(P)
    scratch = torch.empty(max(nb, 1) * num_experts, dtype=torch.int32, device=dev)
    dest = torch.empty(P, dtype=torch.int32, device=dev)
    counts = torch.empty(num_experts, dtype=torch.int32, device=dev)
    starts = torch.empty(num_experts, dtype=torch.int32, device=dev)
    offs = torch.empty(num_experts, dtype=torch.int32, device=dev)
    rc = L.tb_moe_plan(idx.contiguous().data_ptr(), P, num_experts, None, None, scratch.data_ptr(), dest.data_ptr(),
                       counts.data_ptr(), starts.data_ptr(), offs.data_ptr(), capacity, 0,
                       _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "moe_plan")
    return MoePlan(dest, counts, starts, offs, capacity, num_experts, k)


def _ptr_array(tensors):
    arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    return arr


def _gather_raw(x, plan: MoePlan, scale):
    buf = torch.empty(plan.capacity, x.shape[1], dtype=x.dtype, device=x.device)
    if x.is_meta:
        return buf
    L = _lib.lib()
    P = plan.dest.numel()
    rc = L.tb_moe_gather(x.data_ptr(), plan.dest.data_ptr(), _lib.ptr(scale), _ptr_array([buf]), 1, P, plan.top_k,
                         x.shape[1], plan.capacity, _lib.dtype_code(x.dtype), _lib.stream_ptr())
    _lib.check(rc, "moe_gather")
    rc = L.tb_moe_zero_pad(buf.data_ptr(), plan.starts.data_ptr(), plan.counts.data_ptr(), plan.offs.data_ptr(),
                           plan.num_experts, x.shape[1], plan.capacity, _lib.dtype_code(x.dtype), _lib.stream_ptr())
    _lib.check(rc, "moe_zero_pad")
    return buf


def _combine_raw(buf, plan: MoePlan, w, base, T):
    out = torch.empty(T, buf.shape[1], dtype=buf.dtype, device=buf.device)
    if buf.is_meta:
        return out
    rc = _lib.lib().tb_moe_combine(_ptr_array([buf]), 1, plan.dest.data_ptr(), _lib.ptr(w), _lib.ptr(base),
                                   out.data_ptr(), T, plan.top_k, buf.shape[1], plan.capacity,
                                   _lib.dtype_code(buf.dtype), _lib.stream_ptr())
    _lib.check(rc, "moe_combine")
    return out


def _pair_dot_raw(buf, plan: MoePlan, g):
    P = plan.dest.numel()
    d = torch.empty(P, dtype=torch.float32, device=buf.device)
    if buf.is_meta:
        return d
    rc = _lib.lib().tb_moe_pair_dot(_ptr_array([buf]), 1, plan.dest.data_ptr(), g.data_ptr(), d.data_ptr(), P,
                                    plan.top_k, buf.shape[1], plan.capacity, _lib.dtype_code(buf.dtype),
                                    _lib.stream_ptr())
    _lib.check(rc, "moe_pair_dot")
    return d


class _PermuteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, plan):
        x = x.contiguous()
        s32 = scale.reshape(-1).float().contiguous() if scale is not None else None
        ctx.plan, ctx.T = plan, x.shape[0]
        ctx.save_for_backward(x if scale is not None else torch.empty(0), s32 if s32 is not None else torch.empty(0))
        ctx.has_scale = scale is not None
        ctx.scale_shape = scale.shape if scale is not None else None
        return _gather_raw(x, plan, s32)

    @staticmethod
    def backward(ctx, g):
        x, s32 = ctx.saved_tensors
        g = g.contiguous()
        dx = _combine_raw(g, ctx.plan, s32 if ctx.has_scale else None, None, ctx.T)
        ds = None
        if ctx.has_scale:
            ds = _pair_dot_raw(g, ctx.plan, x).view(ctx.scale_shape)
        return dx, ds, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buf, w, base, plan, T):
        buf = buf.contiguous()
        w32 = w.reshape(-1).float().contiguous() if w is not None else None
        ctx.plan = plan
        ctx.save_for_backward(buf if w is not None else torch.empty(0), w32 if w32 is not None else torch.empty(0))
        ctx.has_w, ctx.has_base = w is not None, base is not None
        ctx.w_shape = w.shape if w is not None else None
        return _combine_raw(buf, plan, w32, base.contiguous() if base is not None else None, T)

    @staticmethod
    def backward(ctx, g):
        buf, w32 = ctx.saved_tensors
        g = g.contiguous()
        dbuf = _gather_raw(g, ctx.plan, w32 if ctx.has_w else None)
        dw = _pair_dot_raw(buf, ctx.plan, g).view(ctx.w_shape) if ctx.has_w else None
        return dbuf, dw, (g if ctx.has_base else None), None, None


def permute(x: torch.Tensor, plan: MoePlan, scale: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, D] → padded expert-major [cap, D]; `scale` [T, k] multiplies every routed copy."""
    if not _on_device(x):
        buf = x.new_zeros(plan.capacity, x.shape[1])
        rows = x.repeat_interleave(plan.top_k, dim=0)
        if scale is not None:
            rows = (rows.float() * scale.reshape(-1, 1).float()).to(x.dtype)
        return buf.index_copy(0, plan.dest.long(), rows)
    return _PermuteFn.apply(x, scale, plan)


def combine(buf: torch.Tensor, plan: MoePlan, num_tokens: int, weights: torch.Tensor | None = None,
            base: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = base[t] + Σ_j buf[dest[t,j]] · weights[t,j]."""
    if not _on_device(buf):
        rows = buf[plan.dest.long()].float()
        if weights is not None:
            rows = rows * weights.reshape(-1, 1).float()
        out = rows.view(num_tokens, plan.top_k, -1).sum(1)
        if base is not None:
            out = out + base.float()
        return out.to(buf.dtype)
    return _CombineFn.apply(buf, weights, base, plan, num_tokens)


# ------------------------------------------------------------------------------ grouped GEMM
def grouped_linear_ref(x, w, offs):
    """x [cap, K], w [G, N, K], offs [G] cumulative padded ends → [cap, N] (rows beyond offs[-1] are zero)."""
    out = x.new_zeros(x.shape[0], w.shape[1])
    start = 0
    for g, end in enumerate(offs.tolist()):
        if end > start:
            out[start:end] = (x[start:end].float() @ w[g].float().t()).to(x.dtype)
        start = end
    return out


def _gg_m(a, b, offs, n, b_mn):
    out = torch.empty(a.shape[0], n, dtype=a.dtype, device=a.device)
    G = b.shape[0]
    rc = _lib.lib().tb_grouped_gemm_m(a.data_ptr(), b.data_ptr(), out.data_ptr(), offs.data_ptr(), G, a.shape[0], n,
                                      a.shape[1], int(b_mn), _lib.dtype_code(a.dtype), _lib.shared_status().ptr,
                                      _lib.stream_ptr())
    _lib.check(rc, "grouped_gemm_m")
    return out


def _gg_k(a, b, offs, G):
    out = torch.empty(G, a.shape[1], b.shape[1], dtype=a.dtype, device=a.device)
    rc = _lib.lib().tb_grouped_gemm_k(a.data_ptr(), b.data_ptr(), out.data_ptr(), offs.data_ptr(), G, a.shape[0],
                                      a.shape[1], b.shape[1], _lib.dtype_code(a.dtype), 0, _lib.shared_status().ptr,
                                      _lib.stream_ptr())
    _lib.check(rc, "grouped_gemm_k")
    return out


class _GroupedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, offs):
        x, w = x.contiguous(), w.contiguous()
        ctx.save_for_backward(x, w, offs)
        from titan_b200.ops.registry import ops

        return ops.grouped_gemm_m(x, w, offs, w.shape[1], False)

    @staticmethod
    def backward(ctx, g):
        x, w, offs = ctx.saved_tensors
        g = g.contiguous()
        dx = dw = None
        from titan_b200.ops.registry import ops

        if ctx.needs_input_grad[0]:
            dx = ops.grouped_gemm_m(g, w, offs, w.shape[2], True)   # dy · W[g]   (W stored [N, K] = "[K', N']")
        if ctx.needs_input_grad[1]:
            dw = ops.grouped_gemm_k(g, x, offs, w.shape[0])         # dyᵀ · x per group
        return dx, dw, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
    """Per-expert ``x_g @ w[g].T`` over the padded expert-major layout (tcgen05 grouped GEMM on CUDA).

    Rows at or beyond ``offs[-1]`` are unused capacity: forward leaves them unwritten and backward ignores
    them, so callers must not read them (the MoE path never does: `combine` only follows `dest`)."""
    if not _on_device(x) or x.dtype not in (torch.bfloat16, torch.float16):
        return grouped_linear_ref(x, w, offs)
    return _GroupedLinearFn.apply(x, w, offs)
