"""GEMMs fused with their collective over NVLink peer memory (Python side of `csrc/comm/fused_comm.cu`).

* `all_gather_matmul(a_shard, b)`      – ``concat_ranks(a_shard) @ b.T`` in ONE kernel: a few copier CTAs pull
  every remote shard across NVLink exactly once (bulk async copies, ring order) into a local buffer and hand
  128-row chunks to the GEMM CTAs through flags; the GEMM starts on the local shard at once and consumes
  remote chunks as they land.
* `all_gather_weight_matmul(x, w_shard)` – ``x @ concat_ranks(w_shard).T``: FSDP weight shards are gathered
  inside the first GEMM that consumes them (same mechanism on the B operand, 256-row chunks).
* `matmul_reduce_scatter(a, b)`        – partial ``a @ b.T`` tiles are stored into the owner's staging slot as
  they leave tensor memory; the owner sums the `world` partials once all flags have arrived.
* `castscale_reduce_scatter(bucket, scale)` – gradient bucket reduce-scatter reading peers' buckets directly,
  summing in fp32, scaling and casting in one pass.

Each op has an unfused NCCL + library baseline (`*_baseline`) with identical semantics; tests compare the
two and benchmarks report both.  Buffers live in per-group symmetric workspaces; two staging slots
alternate so a call never waits for the previous call's readers.

Parity: `npu_all_gather_base_mm` / `npu_mm_reduce_scatter_base`
(torchtitan_npu/patches/torch/micro_pipeline_tp.py:35-105) and the FSDP2 collectives.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from titan_b200.ops import _lib
from titan_b200.parallel.symm_mem import SymmWorkspace, get_workspace

__all__ = ["enable_for_group", "enabled_group", "all_gather_matmul", "all_gather_matmul_baseline",
           "all_gather_weight_matmul", "matmul_reduce_scatter", "matmul_reduce_scatter_baseline",
           "castscale_reduce_scatter", "castscale_reduce_scatter_baseline"]

_STATE = {"group": None}
# channels of the workspace flag region
CH_AG_READY, CH_AG_DONE, CH_RS_READY, CH_RS_DONE, CH_GRAD_READY, CH_GRAD_DONE, CH_AGB_READY, CH_AGB_DONE = range(8)


def enable_for_group(group) -> None:
    _STATE["group"] = group


def enabled_group():
    return _STATE["group"]


class _Slots:
    """Two alternating staging slots in a workspace; reuse of a slot waits for the readers of its last use."""

    def __init__(self, ws: SymmWorkspace, slot_bytes: int, ready_ch: int, done_ch: int, base: int = 0):
        self.ws, self.slot_bytes, self.ready_ch, self.done_ch, self.base = ws, slot_bytes, ready_ch, done_ch, base
        self.calls = 0
        self.last_done = [0, 0]

    def acquire(self):
        slot = self.calls & 1
        self.calls += 1
        if self.last_done[slot]:
            self.ws.wait(self.done_ch, self.last_done[slot])
        return slot, self.base + slot * self.slot_bytes

    def release(self, slot: int):
        e = self.ws.next_epoch(self.done_ch)
        self.ws.signal(self.done_ch, e)
        self.last_done[slot] = e


_SLOT_CACHE: dict = {}


def _slots(group, tag: str, slot_bytes: int, ready_ch: int, done_ch: int) -> _Slots:
    slot_bytes = (slot_bytes + 1023) // 1024 * 1024
    ws = get_workspace(group, 2 * slot_bytes, tag)
    key = (id(ws), tag)
    s = _SLOT_CACHE.get(key)
    if s is None or s.slot_bytes < slot_bytes or s.ws is not ws:
        s = _Slots(ws, (ws.nbytes - 4096) // 2 // 1024 * 1024, ready_ch, done_ch)
        _SLOT_CACHE[key] = s
    return s


_CHUNK_FLAGS: dict = {}


def _chunk_flags(ws: SymmWorkspace, tag: str, n: int) -> torch.Tensor:
    """Local hand-off state between copier CTAs and GEMM CTAs: ``n`` chunk flags (zeroed once; epochs only grow)
    followed by ``n`` piece counters (the copier that delivers a chunk's last piece resets its counter)."""
    key = (id(ws), tag, n)
    t = _CHUNK_FLAGS.get(key)
    if t is None:
        t = torch.zeros(2 * n, dtype=torch.int32, device=ws.device)
        _CHUNK_FLAGS[key] = t
    return t


# ------------------------------------------------------------------------------ all-gather → GEMM
def all_gather_matmul_baseline(a_shard, b, group):
    world = dist.get_world_size(group)
    full = torch.empty(world * a_shard.shape[0], a_shard.shape[1], dtype=a_shard.dtype, device=a_shard.device)
    dist.all_gather_into_tensor(full, a_shard.contiguous(), group=group)
    return full @ b.t()


def all_gather_matmul(a_shard: torch.Tensor, b: torch.Tensor, group=None, return_gathered: bool = False):
    """``concat_ranks(a_shard) @ b.T`` → [world·m_shard, N].  a_shard [m_shard, K], b [N, K]; m_shard % 128 == 0.

    ``return_gathered``: also return the gathered operand [world·m_shard, K] (the kernel's copier CTAs build it
    anyway; sequence-parallel linears reuse it for their other projections and for the weight gradient)."""
    group = group or _STATE["group"]
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    m_shard, K = a_shard.shape
    N = b.shape[0]
    if not a_shard.is_cuda or m_shard % 128 or K % 8 or N % 8 or a_shard.dtype not in (torch.bfloat16, torch.float16):
        full = torch.empty(world * m_shard, K, dtype=a_shard.dtype, device=a_shard.device)
        dist.all_gather_into_tensor(full, a_shard.contiguous(), group=group)
        out = full @ b.t()
        return (out, full) if return_gathered else out
    nbytes = m_shard * K * a_shard.element_size()
    s = _slots(group, "ag", nbytes, CH_AG_READY, CH_AG_DONE)
    ws = s.ws
    slot, off = s.acquire()
    ws.view(off, (m_shard, K), a_shard.dtype).copy_(a_shard)
    epoch = ws.next_epoch(CH_AG_READY)
    ws.signal(CH_AG_READY, epoch)
    out = torch.empty(world * m_shard, N, dtype=a_shard.dtype, device=a_shard.device)
    gathered = torch.empty(world * m_shard, K, dtype=a_shard.dtype, device=a_shard.device)
    b = b.contiguous()
    rc = _lib.lib().tb_ag_gemm(ws.ptr_array(off), b.data_ptr(), out.data_ptr(), gathered.data_ptr(),
                               _chunk_flags(ws, "ag", world * m_shard // 128).data_ptr(), world * m_shard, N, K,
                               m_shard, 0, _lib.dtype_code(a_shard.dtype), rank, world,
                               ws.channel_flags_ptr(CH_AG_READY), epoch, _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "ag_gemm")
    s.release(slot)
    if return_gathered:
        # the kernel copies the REMOTE shards; the own shard is read in place
        gathered[rank * m_shard: (rank + 1) * m_shard].copy_(a_shard)
        return out, gathered
    return out


def all_gather_weight_matmul(x: torch.Tensor, w_shard: torch.Tensor, group=None) -> torch.Tensor:
    """``x @ concat_ranks(w_shard).T`` → [M, world·n_shard].  x [M, K], w_shard [n_shard, K]; n_shard % 256 == 0."""
    group = group or _STATE["group"]
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    n_shard, K = w_shard.shape
    M = x.shape[0]
    if not x.is_cuda or n_shard % 256 or K % 8 or x.dtype not in (torch.bfloat16, torch.float16):
        full = torch.empty(world * n_shard, K, dtype=w_shard.dtype, device=w_shard.device)
        dist.all_gather_into_tensor(full, w_shard.contiguous(), group=group)
        return x @ full.t()
    nbytes = n_shard * K * w_shard.element_size()
    s = _slots(group, "agb", nbytes, CH_AGB_READY, CH_AGB_DONE)
    ws = s.ws
    slot, off = s.acquire()
    ws.view(off, (n_shard, K), w_shard.dtype).copy_(w_shard)
    epoch = ws.next_epoch(CH_AGB_READY)
    ws.signal(CH_AGB_READY, epoch)
    out = torch.empty(M, world * n_shard, dtype=x.dtype, device=x.device)
    gathered = torch.empty(world * n_shard, K, dtype=x.dtype, device=x.device)
    x = x.contiguous()
    rc = _lib.lib().tb_ag_b_gemm(x.data_ptr(), ws.ptr_array(off), out.data_ptr(), gathered.data_ptr(),
                                 _chunk_flags(ws, "agb", world * n_shard // 256).data_ptr(), M, world * n_shard, K,
                                 n_shard, _lib.dtype_code(x.dtype), rank, world, ws.channel_flags_ptr(CH_AGB_READY),
                                 epoch, _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "ag_b_gemm")
    s.release(slot)
    return out


# ------------------------------------------------------------------------------ GEMM → reduce-scatter
def matmul_reduce_scatter_baseline(a, b, group):
    world = dist.get_world_size(group)
    full = a @ b.t()
    out = torch.empty(full.shape[0] // world, full.shape[1], dtype=full.dtype, device=full.device)
    dist.reduce_scatter_tensor(out, full, group=group)
    return out


_COUNTERS: dict = {}


def matmul_reduce_scatter(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """``reduce_scatter_rows(a @ b.T)`` → [M / world, N].  a [M, K_local], b [N, K_local]."""
    group = group or _STATE["group"]
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    M, K = a.shape
    N = b.shape[0]
    if not a.is_cuda or M % (128 * world) or K % 8 or N % 8 or a.dtype not in (torch.bfloat16, torch.float16):
        return matmul_reduce_scatter_baseline(a, b, group)
    m_shard = M // world
    nbytes = world * m_shard * N * a.element_size()
    s = _slots(group, "rs", nbytes, CH_RS_READY, CH_RS_DONE)
    ws = s.ws
    slot, off = s.acquire()
    # flags of the two slots must not alias: slot 1 uses the upper half of the channel's 8 entries only when
    # world <= 4; otherwise epochs keep them apart (a slot's epoch is always newer than its previous use)
    epoch = ws.next_epoch(CH_RS_READY)
    key = (id(ws), a.device.index)
    if key not in _COUNTERS:
        _COUNTERS[key] = torch.zeros(8, dtype=torch.int32, device=a.device)
    a, b = a.contiguous(), b.contiguous()
    L = _lib.lib()
    rc = L.tb_gemm_rs(a.data_ptr(), b.data_ptr(), ws.ptr_array(off), ws.peer_channel_flag_ptrs(CH_RS_READY),
                      _COUNTERS[key].data_ptr(), M, N, K, m_shard, 0, _lib.dtype_code(a.dtype), rank, world, epoch,
                      _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "gemm_rs")
    out = torch.empty(m_shard, N, dtype=a.dtype, device=a.device)
    rc = L.tb_rs_reduce(ws.data_ptr(rank, off), ws.channel_flags_ptr(CH_RS_READY), epoch, out.data_ptr(),
                        m_shard * N, world, _lib.dtype_code(a.dtype), _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "rs_reduce")
    s.release(slot)
    return out


# ------------------------------------------------------------------------------ gradient reduce-scatter
def castscale_reduce_scatter_baseline(bucket, scale, out_dtype, group):
    world = dist.get_world_size(group)
    x = bucket.float() * scale
    out = torch.empty(bucket.numel() // world, dtype=torch.float32, device=bucket.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out.to(out_dtype)


def grad_slots(group, nbytes: int) -> _Slots:
    """The two alternating bucket slots of the gradient reduce-scatter in `group`'s symmetric workspace, each at
    least ``nbytes`` large (creating or growing the workspace is a collective over the group)."""
    return _slots(group, "grad", nbytes, CH_GRAD_READY, CH_GRAD_DONE)


def reduce_scatter_slot(slot, numel: int, in_dtype: torch.dtype, out: torch.Tensor, scale: float,
                        nvls: bool = False) -> None:
    """Reduce-scatter a bucket that already sits in a slot from `grad_slots().acquire()`: ``slot`` is
    ``(slots, index, byte offset)``.  Runs on the current stream: publish "my bucket is complete", wait for every
    peer's, reduce this rank's chunk from all buckets into ``out``, then mark the slot as read.  ``nvls``: let the
    NVSwitch add the ranks' buckets (`multimem.ld_reduce` through the multicast address) when the fabric offers it."""
    slots, index, off = slot
    ws = slots.ws
    epoch = ws.next_epoch(CH_GRAD_READY)
    ws.signal(CH_GRAD_READY, epoch)
    ws.wait(CH_GRAD_READY, epoch)
    chunk = numel // ws.world
    esz = torch.empty((), dtype=in_dtype).element_size()
    mc = ws.multicast_ptr(off) if nvls else 0
    if mc and chunk % (16 // esz) == 0:
        _declare_nvls()
        rc = _lib.lib().tb_castscale_rs_nvls(mc + ws.rank * chunk * esz, out.data_ptr(), chunk, float(scale),
                                             _lib.dtype_code(in_dtype), _lib.dtype_code(out.dtype),
                                             _lib.stream_ptr())
        _lib.check(rc, "castscale_rs_nvls")
    else:
        rc = _lib.lib().tb_castscale_rs(ws.ptr_array(off), out.data_ptr(), chunk, ws.rank, ws.world,
                                        float(scale), _lib.dtype_code(in_dtype), _lib.dtype_code(out.dtype),
                                        _lib.stream_ptr())
        _lib.check(rc, "castscale_rs")
    slots.release(index)


_NVLS_DECLARED = False


def _declare_nvls() -> None:
    global _NVLS_DECLARED
    if not _NVLS_DECLARED:
        import ctypes

        P, LL, I, Fl = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
        _lib.declare("tb_castscale_rs_nvls", [P, P, LL, Fl, I, I, P])
        _NVLS_DECLARED = True


def castscale_reduce_scatter(bucket: torch.Tensor, scale: float, out_dtype: torch.dtype = torch.float32,
                             group=None) -> torch.Tensor:
    """``scale · Σ_ranks bucket`` restricted to this rank's chunk, fp32 accumulation, cast to `out_dtype`."""
    group = group or _STATE["group"]
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    n = bucket.numel()
    esz = bucket.element_size()
    if not bucket.is_cuda or n % world or (n // world * esz) % 16 \
            or bucket.dtype not in (torch.bfloat16, torch.float32) \
            or out_dtype not in (torch.bfloat16, torch.float32):
        return castscale_reduce_scatter_baseline(bucket, scale, out_dtype, group)
    s = _slots(group, "grad", n * esz, CH_GRAD_READY, CH_GRAD_DONE)
    ws = s.ws
    slot, off = s.acquire()
    ws.view(off, (n,), bucket.dtype).copy_(bucket.reshape(-1))
    epoch = ws.next_epoch(CH_GRAD_READY)
    ws.signal(CH_GRAD_READY, epoch)
    ws.wait(CH_GRAD_READY, epoch)
    out = torch.empty(n // world, dtype=out_dtype, device=bucket.device)
    rc = _lib.lib().tb_castscale_rs(ws.ptr_array(off), out.data_ptr(), n // world, rank, world, float(scale),
                                    _lib.dtype_code(bucket.dtype), _lib.dtype_code(out_dtype), _lib.stream_ptr())
    _lib.check(rc, "castscale_rs")
    s.release(slot)
    return out
