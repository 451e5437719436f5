"""Expert-parallel MoE dispatch / combine over NVLink peer memory (no NCCL all-to-all, no host sync).

One layer, every rank of the ``ep`` group (E experts, E/P per rank):

  1. counts exchange – each rank puts its per-expert counts into every peer's ``counts_all[P, E]``.
  2. plan            – from ``counts_all`` every rank derives, on the device, the row of each of its
                       (token, slot) pairs inside the OWNER's padded expert-major buffer (rows of lower
                       ranks first, stable inside a rank) — identical arithmetic on all ranks.
  3. dispatch        – ONE kernel permutes and writes the rows straight into the owners' buffers
                       (peer stores); the optional routed score is applied on the way.
  4. experts         – grouped GEMMs on the owner over its local padded layout.
  5. combine         – ONE kernel pulls every token's k expert outputs from the owners (peer loads),
                       applies the weights, adds the shared-expert output and writes the token row.

Backward mirrors it with the same kernels (gather ↔ combine swap roles).  Row capacity per owner is
``capacity_factor · T · k + 128 · E_local``; overflow drops pairs and raises through the status word.

Parity: fuses C9 + C10 + K5 + K6 and C11 + K5 + weighted sum of the reference
(converters/kernels/moe_dispatch.py:156-270, permutation.py:57-143).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from titan_b200.ops import _lib
from titan_b200.ops.moe import ALIGN
from titan_b200.parallel.symm_mem import get_workspace

__all__ = ["moe_forward_ep", "EPContext", "capacity_per_owner"]

CH_COUNTS, CH_DISPATCH, CH_OUT, CH_DONE, CH_BWD_A, CH_BWD_B, CH_BWD_DONE = range(16, 23)
CAPACITY_FACTOR = 4.0  # rows an owner rank can take, over the balanced load (`world` = every pair: dropless)


def set_capacity_factor(factor: float) -> None:
    """Row capacity of an owner rank's receive buffer in multiples of the balanced load (T·k rows).  A routing that
    sends more rows to one owner stops the step with a kernel status (nothing is dropped silently)."""
    global CAPACITY_FACTOR
    if factor < 1.0:
        raise ValueError("expert_parallel_capacity_factor must be at least 1")
    CAPACITY_FACTOR = float(factor)


def capacity_per_owner(pairs: int, e_local: int, world: int, factor: float | None = None) -> int:
    factor = CAPACITY_FACTOR if factor is None else factor
    worst = pairs * world
    cap = min(int(pairs * factor), worst) + (ALIGN - 1) * e_local
    return (cap + ALIGN - 1) // ALIGN * ALIGN


def _put(ws, byte_offset: int, src: torch.Tensor, dst_extra: int = 0) -> None:
    arr = (ctypes.c_void_p * ws.world)(*[ws.data_ptr(r, byte_offset) + dst_extra for r in range(ws.world)])
    rc = _lib.lib().tb_put(arr, ws.world, src.data_ptr(), src.numel() * src.element_size(), _lib.stream_ptr())
    _lib.check(rc, "put")


class EPContext:
    """Per-call routing state shared by the dispatch and combine autograd nodes."""

    def __init__(self, group, T, k, E, D, dtype, device):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.T, self.k, self.E, self.D, self.dtype = T, k, E, D, dtype
        self.e_local = E // self.world
        self.cap = capacity_per_owner(T * k, self.e_local, self.world)
        esz = torch.empty((), dtype=dtype).element_size()
        self.off_counts = 0
        self.off_in = (self.world * E * 4 + 1023) // 1024 * 1024
        self.off_out = self.off_in + self.cap * D * esz
        total = self.off_out + self.cap * D * esz
        self.ws = get_workspace(group, total, "moe")
        self.dest = self.offs_local = self.starts_local = self.totals_local = None

    def in_ptrs(self):
        return self.ws.ptr_array(self.off_in)

    def out_ptrs(self):
        return self.ws.ptr_array(self.off_out)

    def in_view(self):
        return self.ws.view(self.off_in, (self.cap, self.D), self.dtype)

    def out_view(self):
        return self.ws.view(self.off_out, (self.cap, self.D), self.dtype)

    def sync(self, channel: int) -> None:
        self.ws.barrier(channel)

    # ---- step 1 + 2
    def plan(self, idx: torch.Tensor, counts: torch.Tensor) -> None:
        ws, L = self.ws, _lib.lib()
        P = self.T * self.k
        _put(ws, self.off_counts, counts.to(torch.int32).contiguous(), dst_extra=self.rank * self.E * 4)
        self.sync(CH_COUNTS)
        counts_all = ws.view(self.off_counts, (self.world, self.E), torch.int32)
        base = counts_all[: self.rank].sum(0, dtype=torch.int32) if self.rank > 0 else torch.zeros_like(counts_all[0])
        total = counts_all.sum(0, dtype=torch.int32)
        dev = idx.device
        nb = L.tb_moe_plan_blocks(P)
        scratch = torch.empty(max(nb, 1) * self.E, dtype=torch.int32, device=dev)
        self.dest = torch.empty(P, dtype=torch.int32, device=dev)
        mine = torch.empty(self.E, dtype=torch.int32, device=dev)
        starts = torch.empty(self.E, dtype=torch.int32, device=dev)
        offs = torch.empty(self.E, dtype=torch.int32, device=dev)
        rc = L.tb_moe_plan(idx.contiguous().data_ptr(), P, self.E, base.contiguous().data_ptr(), total.data_ptr(),
                           scratch.data_ptr(), self.dest.data_ptr(), mine.data_ptr(), starts.data_ptr(),
                           offs.data_ptr(), self.cap, self.e_local, _lib.shared_status().ptr, _lib.stream_ptr())
        _lib.check(rc, "moe_plan(ep)")
        lo, hi = self.rank * self.e_local, (self.rank + 1) * self.e_local
        self.offs_local = offs[lo:hi].contiguous()
        self.starts_local = starts[lo:hi].contiguous()
        self.totals_local = total[lo:hi].contiguous()

    # ---- kernels over peer buffers
    def push(self, x: torch.Tensor, scale, ptrs) -> None:
        rc = _lib.lib().tb_moe_gather(x.data_ptr(), self.dest.data_ptr(), _lib.ptr(scale), ptrs, self.world,
                                      self.T * self.k, self.k, self.D, self.cap, _lib.dtype_code(x.dtype),
                                      _lib.stream_ptr())
        _lib.check(rc, "moe_gather(ep)")

    def pull(self, ptrs, w, base) -> torch.Tensor:
        out = torch.empty(self.T, self.D, dtype=self.dtype, device=self.dest.device)
        rc = _lib.lib().tb_moe_combine(ptrs, self.world, self.dest.data_ptr(), _lib.ptr(w), _lib.ptr(base),
                                       out.data_ptr(), self.T, self.k, self.D, self.cap, _lib.dtype_code(self.dtype),
                                       _lib.stream_ptr())
        _lib.check(rc, "moe_combine(ep)")
        return out

    def pair_dot(self, ptrs, g: torch.Tensor) -> torch.Tensor:
        d = torch.empty(self.T * self.k, dtype=torch.float32, device=g.device)
        rc = _lib.lib().tb_moe_pair_dot(ptrs, self.world, self.dest.data_ptr(), g.data_ptr(), d.data_ptr(),
                                        self.T * self.k, self.k, self.D, self.cap, _lib.dtype_code(self.dtype),
                                        _lib.stream_ptr())
        _lib.check(rc, "moe_pair_dot(ep)")
        return d

    def _take(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        _declare_take()
        rc = _lib.lib().tb_moe_take(src.data_ptr(), dst.data_ptr(), self.starts_local.data_ptr(),
                                    self.totals_local.data_ptr(), self.offs_local.data_ptr(), self.e_local, self.D,
                                    self.cap, _lib.dtype_code(self.dtype), _lib.stream_ptr())
        _lib.check(rc, "moe_take(ep)")

    def take_local(self, view: torch.Tensor) -> torch.Tensor:
        """The received rows out of the staging buffer, alignment padding zeroed, in ONE pass over the rows in use
        (the buffer is sized for `capacity_factor` times the balanced load; rows past the last expert stay unwritten
        and are never read)."""
        xp = torch.empty_like(view)
        self._take(view, xp)
        return xp

    def publish(self, rows: torch.Tensor, view: torch.Tensor) -> None:
        """Rows in use of a local expert-major tensor → the staging buffer the peers read from."""
        self._take(rows.contiguous(), view)


_TAKE_DECLARED = False


def _declare_take() -> None:
    global _TAKE_DECLARED
    if not _TAKE_DECLARED:
        P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        _lib.declare("tb_moe_take", [P, P, P, P, P, I, I, LL, I, P])
        _TAKE_DECLARED = True


class _EPDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, ep: EPContext):
        x = x.contiguous()
        s32 = scale.reshape(-1).float().contiguous() if scale is not None else None
        ep.push(x, s32, ep.in_ptrs())
        ep.sync(CH_DISPATCH)
        xp = ep.take_local(ep.in_view())
        ctx.ep, ctx.has_scale = ep, scale is not None
        ctx.scale_shape = scale.shape if scale is not None else None
        ctx.save_for_backward(x if scale is not None else torch.empty(0), s32 if s32 is not None else torch.empty(0))
        return xp

    @staticmethod
    def backward(ctx, g):
        ep = ctx.ep
        x, s32 = ctx.saved_tensors
        # owners publish the gradient rows, sources pull their tokens' contributions
        ep.publish(g, ep.in_view())
        ep.sync(CH_BWD_A)
        dx = ep.pull(ep.in_ptrs(), s32 if ctx.has_scale else None, None)
        ds = ep.pair_dot(ep.in_ptrs(), x).view(ctx.scale_shape) if ctx.has_scale else None
        ep.sync(CH_BWD_DONE)
        return dx, ds, None


class _EPCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, yp, w, base, ep: EPContext):
        w32 = w.reshape(-1).float().contiguous() if w is not None else None
        ep.publish(yp, ep.out_view())
        ep.sync(CH_OUT)
        out = ep.pull(ep.out_ptrs(), w32, base.contiguous() if base is not None else None)
        ep.sync(CH_DONE)
        ctx.ep, ctx.has_w, ctx.has_base = ep, w is not None, base is not None
        ctx.w_shape = w.shape if w is not None else None
        ctx.save_for_backward(yp if w is not None else torch.empty(0), w32 if w32 is not None else torch.empty(0))
        return out

    @staticmethod
    def backward(ctx, g):
        ep = ctx.ep
        yp, w32 = ctx.saved_tensors
        g = g.contiguous()
        dw = None
        if ctx.has_w:
            # the weights' gradient needs this layer's expert outputs, which owners still hold
            ep.publish(yp, ep.out_view())
            ep.sync(CH_BWD_B)
            dw = ep.pair_dot(ep.out_ptrs(), g).view(ctx.w_shape)
        ep.push(g, w32 if ctx.has_w else None, ep.in_ptrs())
        ep.sync(CH_BWD_A)
        dyp = ep.take_local(ep.in_view())
        ep.sync(CH_BWD_DONE)
        return dyp, dw, (g if ctx.has_base else None), None


def moe_forward_ep(x2, gate, idx, experts, group, *, base=None, score_before_experts=True):
    """Routed-expert output (+ `base`) for tokens ``x2 [T, D]`` under expert parallelism."""
    T, D = x2.shape
    k = idx.shape[1]
    E = experts.num_experts
    ep = EPContext(group, T, k, E, D, x2.dtype, x2.device)
    counts = torch.bincount(idx.reshape(-1), minlength=E)
    ep.plan(idx, counts)
    if score_before_experts:
        xp = _EPDispatch.apply(x2, gate, ep)
        yp = experts(xp, ep.offs_local, padded=True)
        return _EPCombine.apply(yp, None, base, ep)
    xp = _EPDispatch.apply(x2, None, ep)
    yp = experts(xp, ep.offs_local, padded=True)
    return _EPCombine.apply(yp, gate, base, ep)
