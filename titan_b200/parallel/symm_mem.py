"""Symmetric-memory workspaces for the fused compute+collective kernels.

A `SymmWorkspace` is a byte buffer allocated with CUDA virtual-memory handles that every rank of a
process group has mapped (PyTorch's symmetric-memory allocator does the handle exchange).  It exposes

* ``ptrs[r]``      – device address of rank r's buffer as seen from this rank (peer loads / stores),
* ``flags``        – a small uint32 region at the start of the buffer for epoch flags,
* ``view(...)``    – typed tensor views into the local buffer after the flag region,
* ``signal / wait / barrier`` – time-bounded flag exchange built on `tb_signal` / `tb_wait_flags`.

Epochs are monotonically increasing per channel; a waiter compares ``flag - epoch >= 0``.  Waits give
up after about two seconds and raise `KernelError` at the next status check: kernels never hang on a
peer that went away.

The reference has no counterpart (its fused collectives are vendor ops,
patches/torch/micro_pipeline_tp.py:114-144); this is the plumbing role of its dispatch shim.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from titan_b200.ops import _lib

__all__ = ["SymmWorkspace", "get_workspace", "FLAG_BYTES", "release_all"]

FLAG_BYTES = 4096          # 1024 uint32 flags = 128 channels x 8 ranks
CHANNEL_STRIDE = 8
_WORKSPACES: dict = {}


class SymmWorkspace:
    def __init__(self, group, nbytes: int, device: torch.device | None = None):
        import torch.distributed._symmetric_memory as symm

        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("peer-memory kernels address at most 8 ranks (one NVSwitch domain)")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + FLAG_BYTES + 255) // 256 * 256
        self.buf = symm.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm.rendezvous(self.buf, group)
        # buffer_ptrs are allocation bases; the tensor may sit at an offset inside the allocation
        off = self.buf.data_ptr() - int(self.handle.buffer_ptrs[self.rank])
        if off < 0 or off + self.nbytes > int(self.handle.buffer_size):
            raise RuntimeError("symmetric buffer does not lie inside the rendezvoused allocation")
        self.ptrs = [int(p) + off for p in self.handle.buffer_ptrs]
        # multicast address of the same bytes on every rank (0 when the fabric has no NVLink multicast): loads through
        # it with `multimem.ld_reduce` return the sum over the ranks, computed inside the switch
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.mc_base = mc + off if mc else 0
        self.flags = self.buf[:FLAG_BYTES].view(torch.int32)
        self._epochs: dict[int, int] = {}
        dist.barrier(group=group)

    # ---- addressing
    def data_ptr(self, rank: int, byte_offset: int = 0) -> int:
        return self.ptrs[rank] + FLAG_BYTES + byte_offset

    def multicast_ptr(self, byte_offset: int = 0) -> int:
        """Multicast address of data byte ``byte_offset`` (0 = no multicast support)."""
        return self.mc_base + FLAG_BYTES + byte_offset if self.mc_base else 0

    def ptr_array(self, byte_offset: int = 0):
        return (ctypes.c_void_p * self.world)(*[self.data_ptr(r, byte_offset) for r in range(self.world)])

    def flag_ptr_array(self):
        return (ctypes.c_void_p * self.world)(*[self.ptrs[r] for r in range(self.world)])

    def local_flags_ptr(self) -> int:
        return self.ptrs[self.rank]

    def view(self, byte_offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        n = int(torch.tensor(shape).prod().item()) if len(shape) else 1
        nb = n * torch.empty((), dtype=dtype).element_size()
        if FLAG_BYTES + byte_offset + nb > self.nbytes:
            raise ValueError(f"workspace too small: need {FLAG_BYTES + byte_offset + nb} B, have {self.nbytes} B")
        return self.buf[FLAG_BYTES + byte_offset: FLAG_BYTES + byte_offset + nb].view(dtype).view(*shape)

    # ---- flags
    def next_epoch(self, channel: int) -> int:
        e = self._epochs.get(channel, 0) + 1
        self._epochs[channel] = e
        return e & 0xFFFFFFFF

    def signal(self, channel: int, epoch: int) -> None:
        """Set flag[channel][this rank] = epoch on every rank (ordered after prior work of the stream)."""
        rc = _lib.lib().tb_signal(self.flag_ptr_array(), self.world, channel * CHANNEL_STRIDE + self.rank, epoch,
                                  _lib.stream_ptr())
        _lib.check(rc, "signal")

    def wait(self, channel: int, epoch: int) -> None:
        """Block the stream until every rank's flag of `channel` reached `epoch` (bounded)."""
        rc = _lib.lib().tb_wait_flags(self.local_flags_ptr(), channel * CHANNEL_STRIDE, self.world, epoch,
                                      _lib.shared_status().ptr, _lib.stream_ptr())
        _lib.check(rc, "wait_flags")

    def barrier(self, channel: int) -> int:
        e = self.next_epoch(channel)
        self.signal(channel, e)
        self.wait(channel, e)
        return e

    def channel_flags_ptr(self, channel: int) -> int:
        return self.local_flags_ptr() + channel * CHANNEL_STRIDE * 4

    def peer_channel_flag_ptrs(self, channel: int):
        return (ctypes.c_void_p * self.world)(*[self.ptrs[r] + channel * CHANNEL_STRIDE * 4
                                                for r in range(self.world)])


def get_workspace(group, nbytes: int, tag: str = "default") -> SymmWorkspace:
    """Workspace cache keyed by (group, tag); grown (re-created collectively) when too small."""
    key = (id(group), tag)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.nbytes < nbytes + FLAG_BYTES:
        if ws is not None:
            torch.cuda.synchronize()
            dist.barrier(group=group)
        ws = SymmWorkspace(group, max(nbytes, 1 << 20))
        _WORKSPACES[key] = ws
    return ws


def release_all() -> None:
    _WORKSPACES.clear()
