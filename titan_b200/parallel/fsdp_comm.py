"""FSDP2 collectives over NVLink peer memory (``parallelism.fsdp_reduce_scatter``, ``parallelism.fsdp_all_gather``).

Parameter all-gather (`PeerMemoryAllGather`): FSDP2 writes this rank's shards into its chunk of a gather buffer and
calls an all-gather; here the buffer lives in symmetric memory and every rank PULLS the other chunks with plain
asynchronous device-to-device copies, which run on the copy engines.  No SM is taken from the GEMMs that run while
the next layer's weights arrive (an NCCL all-gather holds a few dozen CTAs for its whole duration), and the bytes
cross NVLink once, at copy-engine rate.  Three buffer slots rotate; a slot is rewritten only after every peer has
signalled that it pulled its chunk.

Gradient reduce-scatter (`PeerMemoryReduceScatter`):

Stock FSDP2 reduces gradients in three passes per parameter group: the bf16 gradients are copied AND cast into one
fp32 bucket, NCCL reduce-scatters that bucket (4 bytes per element on the wire, kernels that hold SMs while the
backward GEMMs run), and the fp32 result is handed on.  `PeerMemoryReduceScatter` plugs into FSDP2's communication
hook (`FSDPModule.set_custom_reduce_scatter`) and shortens this to

    copy-in  bf16 gradients → bf16 bucket that lives in symmetric memory (no cast, 2 bytes per element)
    reduce   ONE kernel reads this rank's chunk of every peer's bucket with plain peer loads, adds in fp32,
             scales and writes the fp32 (or bf16) shard                              (`tb_castscale_rs`)

so half the bytes cross NVLink, the cast pass disappears and the sum is still accumulated in fp32 from the same
bf16 inputs NCCL would have been given.  Two bucket slots alternate; a slot is reused only after every peer has
signalled that it finished reading it (epoch flags, bounded waits that report through the kernel status word).

FSDP2 asks the hook for memory twice per reduction (`allocate`: first the bucket, then the output) and both
requests name the reduce dtype; the bucket is handed out in the wire dtype (the dtype of the gradients) instead.
On CPU / gloo and for reductions the kernel does not cover (other dtypes, a pre-multiplied NCCL op) the hook
falls back to a library reduce-scatter with the same result.

Parity: the FSDP2 collectives the reference inherits (torchtitan_npu/models/deepseek_v32/parallelize.py:255-284).
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.fsdp._fully_shard._fsdp_api import AllGather, ReduceScatter

__all__ = ["PeerMemoryReduceScatter", "PeerMemoryAllGather", "install_peer_reduce_scatter", "install_peer_all_gather",
           "peer_reduce_scatter_wanted", "max_bucket_numel"]


class PeerMemoryReduceScatter(ReduceScatter):
    def __init__(self, group, wire_dtype: torch.dtype = torch.bfloat16, reserve_numel: int = 0, nvls: bool = False):
        self.group = group
        self.world = dist.get_world_size(group)
        self.wire_dtype = wire_dtype
        self.nvls = nvls               # sum inside the NVSwitch (multimem.ld_reduce) instead of one load per peer
        self._bucket_next = True       # FSDP2 allocates the bucket first, then the output, per reduction
        self._slot = None              # (slots, slot index, byte offset) of the bucket handed out last
        self.calls = 0                 # reductions done by the peer-memory kernel (tests, bench records)
        self.fallback_calls = 0
        if reserve_numel and torch.cuda.is_available():
            from titan_b200.ops import fused_comm

            # size the symmetric workspace once, for the largest parameter group: growing it later is a collective
            fused_comm.grad_slots(group, reserve_numel * torch.empty((), dtype=wire_dtype).element_size())

    # ---- memory
    def allocate(self, size, *, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        numel = math.prod(int(s) for s in size)
        if not self._bucket_next:
            self._bucket_next = True
            return torch.empty(numel, dtype=dtype, device=device)
        self._bucket_next = False
        self._slot = None
        if device.type != "cuda":
            return torch.empty(numel, dtype=self.wire_dtype, device=device)
        from titan_b200.ops import fused_comm

        slots = fused_comm.grad_slots(self.group, numel * torch.empty((), dtype=self.wire_dtype).element_size())
        slot, off = slots.acquire()   # the stream waits here until the peers have finished with this slot's last use
        self._slot = (slots, slot, off)
        return slots.ws.view(off, (numel,), self.wire_dtype)

    # ---- reduction
    def _scale_for(self, op) -> float | None:
        if op == dist.ReduceOp.SUM:
            return 1.0
        if op == dist.ReduceOp.AVG:
            return 1.0 / self.world
        return None   # a pre-multiplied sum object: library path

    def __call__(self, output_tensor: torch.Tensor, input_tensor: torch.Tensor, group, op, async_op: bool = False):
        scale = self._scale_for(op)
        slot = self._slot
        self._slot = None
        kernel_ok = (slot is not None and scale is not None and input_tensor.is_cuda
                     and input_tensor.dtype in (torch.bfloat16, torch.float32)
                     and output_tensor.dtype in (torch.bfloat16, torch.float32)
                     and input_tensor.numel() == output_tensor.numel() * self.world
                     and (output_tensor.numel() * input_tensor.element_size()) % 16 == 0)
        if kernel_ok:
            from titan_b200.ops import fused_comm

            fused_comm.reduce_scatter_slot(slot, input_tensor.numel(), input_tensor.dtype, output_tensor, scale,
                                           nvls=self.nvls)
            self.calls += 1
            return None
        if slot is not None:
            slot[0].release(slot[1])
        self.fallback_calls += 1
        wide = input_tensor if input_tensor.dtype == output_tensor.dtype else input_tensor.to(output_tensor.dtype)
        return dist.reduce_scatter_tensor(output=output_tensor, input=wide, group=group, op=op, async_op=async_op)


class PeerMemoryAllGather(AllGather):
    """FSDP2 all-gather as copy-engine pulls from the peers' symmetric buffers (see the module docstring)."""

    SLOTS = 3
    CH_READY, CH_DONE = 8, 9   # flag channels of the workspace (0..7 belong to `ops.fused_comm`)

    def __init__(self, group, reserve_bytes: int = 0):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ws = None
        self.slot_bytes = 0
        self.uses = 0
        self.last_done = [0] * self.SLOTS
        self._pending = None          # (slot, byte offset) handed out by the last `allocate`
        self.calls = self.fallback_calls = 0
        if reserve_bytes and torch.cuda.is_available():
            self._ensure(reserve_bytes)

    def _ensure(self, nbytes: int) -> None:
        from titan_b200.parallel.symm_mem import get_workspace

        need = (nbytes + 1023) // 1024 * 1024
        if self.ws is None or need > self.slot_bytes:
            self.slot_bytes = need
            self.ws = get_workspace(self.group, self.SLOTS * need, "fsdp_ag")   # collective when it (re)allocates
            self.last_done = [0] * self.SLOTS

    def allocate(self, size, *, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        numel = math.prod(int(s) for s in size)
        self._pending = None
        if device.type != "cuda":
            return torch.empty(numel, dtype=dtype, device=device)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        self._ensure(nbytes)
        slot = self.uses % self.SLOTS
        self.uses += 1
        if self.last_done[slot]:
            self.ws.wait(self.CH_DONE, self.last_done[slot])   # every peer has pulled what this slot held before
        off = slot * self.slot_bytes
        self._pending = (slot, off)
        return self.ws.view(off, (numel,), dtype)

    def __call__(self, output_tensor: torch.Tensor, input_tensor: torch.Tensor, group, async_op: bool = False):
        pend = self._pending
        self._pending = None
        if pend is None or not output_tensor.is_cuda:
            self.fallback_calls += 1
            return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group, async_op=async_op)
        from titan_b200.ops import _lib

        slot, off = pend
        ws = self.ws
        chunk = input_tensor.numel() * input_tensor.element_size()
        ready = ws.next_epoch(self.CH_READY)
        ws.signal(self.CH_READY, ready)      # my chunk is in place (the stream is ordered after FSDP's copy-in)
        ws.wait(self.CH_READY, ready)        # ... and so is everybody else's
        L, st = _lib.lib(), _lib.stream_ptr()
        for d in range(1, self.world):       # ring order: spreads the pulls over the peers
            r = (self.rank + d) % self.world
            rc = L.tb_peer_copy(ws.data_ptr(self.rank, off + r * chunk), ws.data_ptr(r, off + r * chunk), chunk, st)
            _lib.check(rc, "peer_copy")
        done = ws.next_epoch(self.CH_DONE)
        ws.signal(self.CH_DONE, done)        # I no longer read the peers' copies of this slot
        self.last_done[slot] = done
        self.calls += 1
        return None


def max_bucket_numel(model: nn.Module, world: int) -> int:
    """Largest gradient bucket FSDP2 will build for `model`: per FSDP parameter group, every parameter padded on
    dim 0 to a multiple of ``world``."""
    from torch.distributed.fsdp import FSDPModule

    best = 0
    seen: set[int] = set()
    # inner groups first: a parameter belongs to the innermost FSDP module that contains it
    mods = [m for m in model.modules() if isinstance(m, FSDPModule)]
    for m in reversed(mods):
        total = 0
        for p in m.parameters():
            if id(p) in seen:
                continue
            seen.add(id(p))
            shape = tuple(p.shape)
            rows = shape[0] if shape else 1
            rest = math.prod(shape[1:]) if len(shape) > 1 else 1
            total += -(-rows // world) * world * rest
        best = max(best, total)
    return best


def peer_reduce_scatter_wanted(setting: str, dp_mesh, device_type: str) -> bool:
    """``auto``: on for CUDA jobs whose FSDP group sits inside one NVSwitch domain (2..8 ranks of one node)."""
    if setting == "nccl":
        return False
    shard_mesh = dp_mesh if dp_mesh.ndim == 1 else dp_mesh[dp_mesh.mesh_dim_names[-1]]
    n = shard_mesh.size()
    import os

    one_node = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1"))) == \
        int(os.environ.get("WORLD_SIZE", "1"))
    ok = device_type == "cuda" and 2 <= n <= 8 and one_node
    if setting in ("peer_memory", "nvls") and not ok and device_type == "cuda":
        raise ValueError(f"fsdp_reduce_scatter={setting} needs an FSDP group of 2..8 GPUs on one node")
    return ok or setting in ("peer_memory", "nvls")


def install_peer_all_gather(model: nn.Module, dp_mesh, param_dtype: torch.dtype) -> PeerMemoryAllGather | None:
    """Give every FSDP module of `model` whose shard group is ``dp_mesh``'s shard axis the copy-engine all-gather."""
    from torch.distributed.fsdp import FSDPModule

    shard_mesh = dp_mesh if dp_mesh.ndim == 1 else dp_mesh[dp_mesh.mesh_dim_names[-1]]
    group = shard_mesh.get_group()
    world = shard_mesh.size()
    if world < 2:
        return None
    esize = torch.empty((), dtype=param_dtype).element_size()
    comm = PeerMemoryAllGather(group, reserve_bytes=max_bucket_numel(model, world) * esize)
    for m in model.modules():
        if not isinstance(m, FSDPModule) or getattr(m, "_keeps_library_collectives", False):
            continue
        pg = getattr(m._get_fsdp_state(), "_fsdp_param_group", None)
        other = getattr(pg.mesh_info, "shard_process_group", None) if pg is not None else None
        if other is None or other.group_name != group.group_name:
            continue
        m.set_custom_all_gather(comm)
    return comm


def install_peer_reduce_scatter(model: nn.Module, dp_mesh, wire_dtype: torch.dtype,
                                nvls: bool = False) -> PeerMemoryReduceScatter | None:
    """Give every FSDP module of `model` whose shard group is ``dp_mesh``'s shard axis the peer-memory hook."""
    from torch.distributed.fsdp import FSDPModule

    shard_mesh = dp_mesh if dp_mesh.ndim == 1 else dp_mesh[dp_mesh.mesh_dim_names[-1]]
    group = shard_mesh.get_group()
    world = shard_mesh.size()
    if world < 2:
        return None
    comm = PeerMemoryReduceScatter(group, wire_dtype, reserve_numel=max_bucket_numel(model, world), nvls=nvls)
    for m in model.modules():
        if not isinstance(m, FSDPModule) or getattr(m, "_keeps_library_collectives", False):
            continue
        state = m._get_fsdp_state()
        pg = getattr(state, "_fsdp_param_group", None)
        other = getattr(pg.mesh_info, "shard_process_group", None) if pg is not None else None
        if other is None or other.group_name != group.group_name:
            continue   # e.g. experts sharded on their own mesh keep the library collective
        m.set_custom_reduce_scatter(comm)
    return comm
