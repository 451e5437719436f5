"""Kernel status word → training loop.

The sm_100a kernels never trap: a bounded wait that ran out (a peer flag, a TMA or tensor-memory barrier), an
expert-parallel buffer that overflowed its row capacity or a failed index check is recorded as a code in one int32
per device (`titan_b200.ops._lib.shared_status`) and the kernel returns; the affected output is then incomplete.
`KernelStatusMonitor` makes the trainer see that word:

* every step it queues a non-blocking copy of the word into pinned host memory and inspects the copy queued one
  step earlier (by then complete), so a failure stops training at most one step late without adding a host sync;
* at log steps and before a checkpoint is written it reads the word with a synchronising copy, so a corrupt step
  is never logged as healthy nor saved.

A non-zero word raises `KernelError` with the decoded text and clears the word.
"""

from __future__ import annotations

from collections.abc import Callable

import torch

__all__ = ["KernelStatusMonitor"]


def _default_status_tensor():
    if not torch.cuda.is_available():
        return None
    from titan_b200.ops import _lib

    if not _lib.available():
        return None
    return _lib.shared_status().t


class KernelStatusMonitor:
    def __init__(self, status_tensor_fn: Callable[[], torch.Tensor | None] = _default_status_tensor):
        self._status_tensor_fn = status_tensor_fn
        self._pending: tuple[torch.Tensor, object] | None = None   # (host copy, event) queued at the previous step

    def _raise(self, code: int, where: str) -> None:
        from titan_b200.ops._lib import _STATUS_TEXT, KernelError

        t = self._status_tensor_fn()
        if t is not None:
            t.zero_()
        self._pending = None
        raise KernelError(f"{where}: a kernel reported '{_STATUS_TEXT.get(code, code)}' (status {code}); the outputs "
                          "of that step are incomplete")

    def poll(self, where: str = "train step") -> None:
        """Non-blocking: look at the copy queued by the previous call, then queue a new one."""
        t = self._status_tensor_fn()
        if t is None:
            return
        if self._pending is not None:
            host, ev = self._pending
            if ev is None or ev.query():
                code = int(host.item())
                self._pending = None
                if code != 0:
                    self._raise(code, where)
            else:
                return  # the earlier copy has not landed yet: keep it, queue nothing new
        if t.is_cuda:
            host = torch.empty(1, dtype=t.dtype, pin_memory=True)
            host.copy_(t, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._pending = (host, ev)
        else:
            self._pending = (t.clone(), None)

    def check(self, where: str) -> None:
        """Blocking: read the word now."""
        t = self._status_tensor_fn()
        if t is None:
            return
        code = int(t.item())
        if code != 0:
            self._raise(code, where)
