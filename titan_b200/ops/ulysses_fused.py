"""Ulysses head <-> sequence all-to-all fused into the projections on either side of it.

* `proj_all_to_all(x, w, seq_local)` – ``x @ w.T`` whose epilogue stores every 64-column box of the result straight
  into the receive buffer of the rank that owns those heads (peer stores over NVLink; flags tell the owner when a
  source is complete).  x ``[B·S_local, K]`` holds this rank's sequence slice, the result ``[B·S_full, N / cp]`` holds
  this rank's heads over the full sequence.
* `all_to_all_proj(o, w, seq_local)` – the way back fused into the consuming GEMM: ``o [B·S_full, K / cp]`` (this
  rank's heads) is published in symmetric memory; copier CTAs of the GEMM pull the other ranks' head slices of THIS
  rank's rows once into a local buffer while the tensor cores already work on the local slice; result
  ``[B·S_local, N]``.

Both are autograd functions and each one's backward is the other kernel (the exchange is its own transpose).
Without CUDA, or for shapes the kernels do not take, the same results come from `all_to_all_single` + matmul.

Parity: torchtitan_npu/distributed/context_parallel/ulysses_cp.py:28-64 (chunk -> all_to_all -> cat around attention).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from titan_b200.ops import _lib
from titan_b200.ops.fused_comm import _COUNTERS, _chunk_flags, _slots

__all__ = ["proj_all_to_all", "all_to_all_proj", "proj_all_to_all_baseline", "all_to_all_proj_baseline"]

CH_UA_READY, CH_UA_DONE, CH_UG_READY, CH_UG_DONE = 8, 9, 10, 11


# ------------------------------------------------------------------------------------------------ unfused forms
def _heads_to_seq(y: torch.Tensor, seq_local: int, group) -> torch.Tensor:
    """[B·S_local, cp·n] (all heads, my rows) -> [B·S_full, n] (my heads, all rows)."""
    world = dist.get_world_size(group)
    M, N = y.shape
    b, n = M // seq_local, N // world
    send = y.view(b, seq_local, world, n).permute(2, 0, 1, 3).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.permute(1, 0, 2, 3).reshape(b * world * seq_local, n)


def _seq_to_heads(o: torch.Tensor, seq_local: int, group) -> torch.Tensor:
    """[B·S_full, k] (my heads, all rows) -> [cp, B·S_local, k] (every rank's heads, my rows)."""
    world = dist.get_world_size(group)
    rows, k = o.shape
    b = rows // (world * seq_local)
    send = o.view(b, world, seq_local, k).permute(1, 0, 2, 3).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.view(world, b * seq_local, k)


def proj_all_to_all_baseline(x, w, seq_local, group, w_is_kn: bool = False):
    return _heads_to_seq(x @ (w if w_is_kn else w.t()), seq_local, group)


def all_to_all_proj_baseline(o, w, seq_local, group, w_is_kn: bool = False):
    g = _seq_to_heads(o, seq_local, group)
    a = g.permute(1, 0, 2).reshape(g.shape[1], -1)
    return a @ (w if w_is_kn else w.t()), g


# ------------------------------------------------------------------------------------------------ kernels
def _fusable(t: torch.Tensor, seq_local: int) -> bool:
    return t.is_cuda and t.dtype in (torch.bfloat16, torch.float16) and seq_local % 128 == 0


def _scatter(x, w, seq_local, group, w_is_kn: bool):
    """x [M, K] · w -> [M·cp, N / cp]; w is [N, K], or [K, N] when `w_is_kn`."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    M, K = x.shape
    N = w.shape[1] if w_is_kn else w.shape[0]
    if world == 1:
        return x @ (w if w_is_kn else w.t())
    n_shard = N // world
    if not _fusable(x, seq_local) or N % world or n_shard % 64 or K % 8 or M % seq_local:
        return proj_all_to_all_baseline(x, w, seq_local, group, w_is_kn)
    s = _slots(group, "ua2a", M * N * x.element_size(), CH_UA_READY, CH_UA_DONE)
    ws = s.ws
    slot, off = s.acquire()
    epoch = ws.next_epoch(CH_UA_READY)
    key = (id(ws), x.device.index)
    if key not in _COUNTERS:
        _COUNTERS[key] = torch.zeros(8, dtype=torch.int32, device=x.device)
    x, w = x.contiguous(), w.contiguous()
    rc = _lib.lib().tb_gemm_a2a_scatter(x.data_ptr(), w.data_ptr(), ws.ptr_array(off),
                                        ws.peer_channel_flag_ptrs(CH_UA_READY), _COUNTERS[key].data_ptr(), M, N, K,
                                        n_shard, seq_local, 1 if w_is_kn else 0, _lib.dtype_code(x.dtype), rank,
                                        world, epoch, _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "gemm_a2a_scatter")
    ws.wait(CH_UA_READY, epoch)  # every source has delivered its rows of my heads
    out = ws.view(off, (M * world, n_shard), x.dtype).clone()
    s.release(slot)
    return out


def _gather(o, w, seq_local, group, w_is_kn: bool):
    """gather_k(o [M·cp, k]) · w -> ([M, N], gathered [cp, M, k]); w is [N, cp·k], or [cp·k, N] when `w_is_kn`."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    rows, k = o.shape
    M = rows // world
    N = w.shape[1] if w_is_kn else w.shape[0]
    if world == 1:
        return o @ (w if w_is_kn else w.t()), o.view(1, M, k)
    if not _fusable(o, seq_local) or k % 64 or N % 8 or M % seq_local:
        return all_to_all_proj_baseline(o, w, seq_local, group, w_is_kn)
    s = _slots(group, "ug", rows * k * o.element_size(), CH_UG_READY, CH_UG_DONE)
    ws = s.ws
    slot, off = s.acquire()
    ws.view(off, (rows, k), o.dtype).copy_(o)
    epoch = ws.next_epoch(CH_UG_READY)
    ws.signal(CH_UG_READY, epoch)
    out = torch.empty(M, N, dtype=o.dtype, device=o.device)
    gathered = torch.empty(world, M, k, dtype=o.dtype, device=o.device)
    w = w.contiguous()
    rc = _lib.lib().tb_a2a_gather_gemm(ws.ptr_array(off), w.data_ptr(), out.data_ptr(), gathered.data_ptr(),
                                       _chunk_flags(ws, "ug", world * M // 128).data_ptr(), M, N, k, seq_local,
                                       1 if w_is_kn else 0, _lib.dtype_code(o.dtype), rank, world,
                                       ws.channel_flags_ptr(CH_UG_READY), epoch, _lib.shared_status().ptr,
                                       _lib.stream_ptr())
    _lib.check(rc, "a2a_gather_gemm")
    s.release(slot)
    # the kernel copies the REMOTE slices; this rank's own slice of its rows is read in place
    b = M // seq_local
    gathered[rank].copy_(o.view(b, world, seq_local, k)[:, rank].reshape(M, k))
    return out, gathered


# ------------------------------------------------------------------------------------------------ autograd
class _ProjA2A(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, seq_local, group):
        ctx.save_for_backward(x, w)
        ctx.seq_local, ctx.group = seq_local, group
        return _scatter(x, w, seq_local, group, False)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        # dx = gather_heads(g) · w  (w [N, K] is the [contraction, out] layout of this product)
        dx, gathered = _gather(g.contiguous(), w, ctx.seq_local, ctx.group, True)
        # dw rows of owner r = gathered[r]ᵀ · x
        dw = torch.matmul(gathered.transpose(1, 2), x).reshape(w.shape)
        return dx, dw, None, None


class _A2AProj(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, w, seq_local, group):
        out, gathered = _gather(o, w, seq_local, group, False)
        ctx.save_for_backward(gathered, w)
        ctx.seq_local, ctx.group = seq_local, group
        return out

    @staticmethod
    def backward(ctx, g):
        gathered, w = ctx.saved_tensors
        g = g.contiguous()
        # do = scatter_heads(g · w)  (w [N, K] read as [contraction, out])
        do = _scatter(g, w, ctx.seq_local, ctx.group, True)
        world, M, k = gathered.shape
        dw = g.t() @ gathered.permute(1, 0, 2).reshape(M, world * k)
        return do, dw, None, None


def proj_all_to_all(x: torch.Tensor, w: torch.Tensor, seq_local: int, group) -> torch.Tensor:
    """``heads_to_seq(x @ w.T)``: x [B·S_local, K], w [N, K] -> [B·S_full, N / cp]."""
    return _ProjA2A.apply(x, w, seq_local, group)


def all_to_all_proj(o: torch.Tensor, w: torch.Tensor, seq_local: int, group) -> torch.Tensor:
    """``seq_to_heads(o) @ w.T``: o [B·S_full, K / cp], w [N, K] -> [B·S_local, N]."""
    return _A2AProj.apply(o, w, seq_local, group)
