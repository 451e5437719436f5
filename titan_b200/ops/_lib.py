"""ctypes binding of the sm_100a kernel library.

`lib()` returns the loaded ``libtitan_b200.so`` (built in-tree by `titan_b200.csrc.build`).  If the
library is missing on a machine that has a GPU, loading raises: a fused op must never fall back
silently to library math.  Every kernel entry returns an int: 0 = launched, otherwise an error
code (`check`) — kernels themselves report run-time failures (bounded waits that expired, index
checks) through a status word that `StatusWord` owns.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import torch

__all__ = ["lib", "available", "check", "stream_ptr", "ptr", "dtype_code", "StatusWord", "KernelError", "LIB_PATH"]

LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C", "libtitan_b200.so")
_LIB = None

_STATUS_TEXT = {
    1: "TMA full-barrier wait expired",
    2: "empty-barrier wait expired",
    3: "TMEM-full wait expired",
    4: "TMEM-empty wait expired",
    5: "peer flag wait expired",
    6: "index out of bounds (access skipped)",
    7: "invalid arguments",
}


class KernelError(RuntimeError):
    pass


def _declare(L) -> None:
    P, I, LL, F = c_void_p, c_int, c_longlong, c_float
    sig = {
        "tb_rmsnorm_bwd_grid": [I, I],
        "tb_rmsnorm_fwd": [P, P, P, P, I, I, F, I, P],
        "tb_rmsnorm_bwd": [P, P, P, P, P, P, P, I, I, I, P],
        "tb_rope": [P, P, P, P, LL, I, I, I, I, I, I, I, I, P, P],
        "tb_swiglu_fwd": [P, P, P, P, LL, I, LL, LL, F, I, P],
        "tb_swiglu_bwd": [P, P, P, P, P, P, P, LL, I, LL, LL, F, I, P],
        "tb_adam_limits": [P, P, P],
        "tb_adamw_multi": [P, P, P, P, P, P, I, F, F, F, F, F, LL, P, I, I, I, I, I, I, P],
        "tb_cross_entropy_fwd": [P, P, P, P, LL, I, LL, LL, I, P, P],
        "tb_cross_entropy_bwd": [P, P, P, P, P, LL, I, LL, LL, I, P],
        "tb_gemm_bf16": [P, P, P, I, I, I, LL, LL, LL, I, I, I, I, I, I, P, P],
        "tb_gemm_auto": [P, P, P, I, I, I, LL, LL, LL, I, I, I, I, I, I, P, LL, I, P, P],
        "tb_grouped_gemm_m": [P, P, P, P, I, I, I, I, I, I, P, P],
        "tb_grouped_gemm_k": [P, P, P, P, I, I, I, I, I, I, P, P],
        "tb_router_topk": [P, P, P, P, P, P, P, I, I, I, I, I, F, P, P],
        "tb_moe_plan_blocks": [I],
        "tb_moe_plan": [P, I, I, P, P, P, P, P, P, P, I, I, P, P],
        "tb_moe_gather": [P, P, P, P, I, I, I, I, LL, I, P],
        "tb_moe_zero_pad": [P, P, P, P, I, I, LL, I, P],
        "tb_moe_combine": [P, I, P, P, P, P, I, I, I, LL, I, P],
        "tb_moe_pair_dot": [P, I, P, P, P, I, I, I, LL, I, P],
        "tb_signal": [P, I, I, c_uint, P],
        "tb_wait_flags": [P, I, I, c_uint, P, P],
        "tb_ag_gemm": [P, P, P, P, P, I, I, I, I, I, I, I, I, P, c_uint, P, P],
        "tb_ag_b_gemm": [P, P, P, P, P, I, I, I, I, I, I, I, P, c_uint, P, P],
        "tb_gemm_rs": [P, P, P, P, P, I, I, I, I, I, I, I, I, c_uint, P, P],
        "tb_rs_reduce": [P, P, c_uint, P, LL, I, I, P, P],
        "tb_castscale_rs": [P, P, LL, I, I, F, I, I, P],
        "tb_put": [P, I, P, LL, P],
        "tb_peer_copy": [P, P, LL, P],
        "tb_gemm_a2a_scatter": [P, P, P, P, P, I, I, I, I, I, I, I, I, I, c_uint, P, P],
        "tb_a2a_gather_gemm": [P, P, P, P, P, I, I, I, I, I, I, I, I, P, c_uint, P, P],
    }
    for name, args in sig.items():
        fn = getattr(L, name, None)
        if fn is None:
            continue
        fn.argtypes = args
        fn.restype = c_int


class _NoLaunchLibrary:
    """Stands in for the kernel library while shapes are traced on meta tensors: every entry point returns 0."""

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)

        def fn(*args, **kwargs):
            sink = _NO_LAUNCH.get("sink")
            if sink is not None:
                sink(name, args)            # a cost model may price the launch from its name and integer arguments
            return 0

        fn.argtypes, fn.restype = None, None
        return fn


class _NoLaunchStatus:
    ptr = None

    def read(self) -> int:
        return 0

    def raise_if_set(self, what: str) -> None:
        return None


_NO_LAUNCH = {"depth": 0}
_PENDING_DECLARATIONS: dict[str, list] = {}


class no_launch:
    """``with no_launch():`` the wrappers run their device code paths (buffers, saved tensors, autograd nodes) on
    meta tensors and no kernel is launched: `lib()` hands out a stand-in, `stream_ptr()` is 0, the status word is
    inert.  The memory simulator measures a step this way."""

    def __init__(self, on_call=None):
        self.on_call = on_call              # optional ``(entry point name, args)`` callback for every skipped launch

    def __enter__(self):
        _NO_LAUNCH["depth"] += 1
        self._outer_sink = _NO_LAUNCH.get("sink")
        if self.on_call is not None:
            _NO_LAUNCH["sink"] = self.on_call
        return self

    def __exit__(self, *exc):
        _NO_LAUNCH["depth"] -= 1
        _NO_LAUNCH["sink"] = self._outer_sink
        return False


def note_skipped_launch(name: str, args: tuple) -> None:
    """A wrapper that returns early on meta tensors reports the launch it skipped (same form as the stand-in
    library: entry point name and its arguments, pointers may be None)."""
    sink = _NO_LAUNCH.get("sink")
    if sink is not None:
        sink(name, args)


def launches_disabled() -> bool:
    return _NO_LAUNCH["depth"] > 0


def on_device(t: torch.Tensor) -> bool:
    """True for tensors that take the kernel code paths: CUDA tensors, and meta tensors inside `no_launch()`."""
    return t.is_cuda or (t.is_meta and _NO_LAUNCH["depth"] > 0)


def lib():
    global _LIB
    if _NO_LAUNCH["depth"] > 0:
        return _NoLaunchLibrary()
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise KernelError(
                f"{LIB_PATH} is missing: run `python -m titan_b200.csrc.build` (needs nvcc; no GPU required)")
        _LIB = ctypes.CDLL(LIB_PATH)
        _declare(_LIB)
    if _PENDING_DECLARATIONS:
        for name, argtypes in list(_PENDING_DECLARATIONS.items()):
            fn = getattr(_LIB, name)
            fn.argtypes, fn.restype = argtypes, c_int
        _PENDING_DECLARATIONS.clear()
    return _LIB


def declare(name: str, argtypes: list) -> None:
    """Late declaration for entry points added by optional source files."""
    if _NO_LAUNCH["depth"] > 0:
        _PENDING_DECLARATIONS[name] = argtypes   # callers remember "declared": applied when the real library is used
        return
    fn = getattr(lib(), name)
    fn.argtypes = argtypes
    fn.restype = c_int


def launch_count() -> int:
    """Kernels launched by the library in this process."""
    fn = lib().tb_launch_count
    fn.restype = ctypes.c_longlong
    fn.argtypes = []
    return int(fn())


def available() -> bool:
    """True when CUDA is present (the library must then load, or this raises)."""
    if not torch.cuda.is_available():
        return False
    lib()
    return True


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc >= 2000:
        raise KernelError(f"{what}: cuTensorMapEncodeTiled failed with CUresult {rc - 2000}")
    if rc >= 1000:
        raise KernelError(f"{what}: CUDA runtime error {rc - 1000}")
    raise KernelError(f"{what}: {_STATUS_TEXT.get(rc, f'error {rc}')}")


_TLS = threading.local()


def stream_ptr() -> int:
    """Current stream handle; also binds the calling thread to the current device inside the library."""
    if _NO_LAUNCH["depth"] > 0:
        return 0
    dev = torch.cuda.current_device()
    if getattr(_TLS, "device", None) != dev:
        fn = lib().tb_bind_device
        fn.argtypes, fn.restype = [c_int], c_int
        check(fn(dev), "bind_device")
        _TLS.device = dev
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_DTYPE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE[dt]
    except KeyError:
        raise KernelError(f"unsupported dtype {dt}") from None


class StatusWord:
    """A device int32 that kernels write error codes into; `raise_if_set` syncs and checks it."""

    def __init__(self, device=None):
        self.t = torch.zeros(1, dtype=torch.int32, device=device or torch.device("cuda", torch.cuda.current_device()))

    @property
    def ptr(self) -> int:
        return self.t.data_ptr()

    def read(self) -> int:
        return int(self.t.item())

    def raise_if_set(self, what: str) -> None:
        code = self.read()
        if code != 0:
            self.t.zero_()
            raise KernelError(f"{what}: kernel reported '{_STATUS_TEXT.get(code, code)}'")


_STATUS_CACHE: dict[int, StatusWord] = {}


def shared_status() -> StatusWord:
    """One status word per device, checked lazily (e.g. at log steps) to avoid per-op syncs."""
    if _NO_LAUNCH["depth"] > 0:
        return _NoLaunchStatus()
    dev = torch.cuda.current_device()
    if dev not in _STATUS_CACHE:
        _STATUS_CACHE[dev] = StatusWord()
    return _STATUS_CACHE[dev]
