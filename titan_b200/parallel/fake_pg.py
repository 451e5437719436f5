"""Fake process group: one process pretends to be `world_size` ranks.

Every collective returns immediately with shape-correct (uninitialised or input)
data, so model build, converters, parallelisation, one training step and the memory
estimate run on a single CPU process.  Code that uses the *result* of a collective
as a size (expert-parallel split sizes) must branch on `is_fake_process_group`.

Parity: torchtitan_npu/patches/torch/testing/_internal/distributed/fake_pg.py:14-36,
distributed/process_group.py:11-18, scripts/run_train.sh:23-27.
"""

from __future__ import annotations

import torch.distributed as dist

__all__ = ["init_fake_process_group", "is_fake_process_group", "fake_mode_active"]

_ACTIVE = {"fake": False}


def init_fake_process_group(rank: int = 0, world_size: int = 1) -> None:
    from torch.testing._internal.distributed.fake_pg import FakeStore  # registers the "fake" backend

    if dist.is_initialized():
        return
    dist.init_process_group(backend="fake", rank=rank, world_size=world_size, store=FakeStore())
    _ACTIVE["fake"] = True


def fake_mode_active() -> bool:
    return _ACTIVE["fake"] and dist.is_initialized()


def is_fake_process_group(group=None) -> bool:
    if not dist.is_initialized():
        return False
    try:
        backend = dist.get_backend(group)
    except Exception:
        return False
    return str(backend).lower() == "fake"
