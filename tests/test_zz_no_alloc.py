"""Allocation-free RMSNorm backward (`tb_rmsnorm_bwd_noalloc`).

Some hosts of this library cannot let it allocate device memory: the process may have given all of HBM to
its own arena, may be in a latency-critical loop where an allocation call could stall, or may call in from a
runtime that forbids allocation in callbacks.  For them the library exports a variant of the RMSNorm backward
whose partial-sum scratch is a fixed array inside the library image.  This test calls that variant through
its exported C symbol (plain ctypes, as such a host would) and checks it against the regular entry point,
which uses a caller-provided scratch buffer, on two consecutive calls: the second call sees the scratch
contents left by the first and must still be right.

The oracle here is the regular entry point on purpose (both must agree bit for bit); the regular entry point itself is
pinned against an fp32 PyTorch statement of RMSNorm backward in `tests/test_kernels_elementwise_gpu.py`.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_DIM = 8192


def _lib():
    from titan_b200.ops import _lib

    L = _lib.lib()
    fn = L.tb_rmsnorm_bwd_noalloc
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    fn.restype = ctypes.c_int
    err = L.tb_rmsnorm_bwd_noalloc_strerror
    err.argtypes = [ctypes.c_int]
    err.restype = ctypes.c_char_p
    return L, fn, err


def _case(rows, dim, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, dim, device="cuda", generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(dim, device="cuda", generator=g)).to(dtype)
    gy = torch.randn(rows, dim, device="cuda", generator=g).to(dtype)
    return x, w, gy


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_matches_regular_entry_point_twice(cuda_device, dtype):
    from titan_b200.ops import _lib as binding
    from titan_b200.ops.norm import rms_norm_bwd, rms_norm_fwd

    _, fn, err = _lib()
    stream = binding.stream_ptr()
    code = binding.dtype_code(dtype)
    # two different problems back to back: the second runs over whatever the first left in the scratch array
    for rows, dim, seed in [(2000, 4096, 1), (300, 1536, 2)]:
        x, w, gy = _case(rows, dim, dtype, seed)
        _, rstd = rms_norm_fwd(x, w, 1e-5)
        dx_ref, dw_ref = rms_norm_bwd(gy, x, w, rstd)
        dx = torch.empty_like(x)
        dw = torch.empty_like(w)
        before = torch.cuda.memory_allocated()
        rc = fn(gy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, dim,
                code, stream)
        assert rc == 0, err(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before  # nothing was allocated through torch either
        tol = dict(rtol=1e-2, atol=1e-2)
        torch.testing.assert_close(dx.float(), dx_ref.float(), **tol)
        # both entry points sum partial rows in a fixed order but over different CTA counts
        torch.testing.assert_close(dw.float(), dw_ref.float(), rtol=2e-2, atol=2e-2 * max(1.0, rows ** 0.5 / 4))


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch(cuda_device):
    from titan_b200.ops import _lib as binding

    _, fn, err = _lib()
    x = torch.zeros(4, 8, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 4, MAX_DIM + 8, 0,
            binding.stream_ptr())
    assert rc == -1 and b"8192" in err(rc)
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 0, 8, 0,
            binding.stream_ptr())
    assert rc == -2
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 4, 6, 1,
            binding.stream_ptr())
    assert rc == -2  # 6 bf16 elements are not a whole 16-byte vector
