"""tcgen05 GEMM: Python entry points, a `linear` autograd function and oracles.

``gemm(a, b, a_mn=False, b_mn=False)`` computes ``A · B`` for bf16/fp16 operands on the
tcgen05 tensor cores with fp32 accumulation in tensor memory.  Large problems run on CTA pairs
(`csrc/gemm/gemm_pair.cuh`: ``cta_group::2``, 256 x 256 tiles, the last partial wave cut along the
contraction), small ones on the single-CTA engine (`csrc/gemm/gemm_bf16.cu`); ``policy`` forces either.
`a_mn` / `b_mn` say how each operand is *stored* (see that file); `linear(x, w)` uses the
three storage combinations so forward, input-gradient and weight-gradient run without transposes:

    y  = x · wᵀ      gemm(x,  w)                       (both K-major)
    dx = dy · w      gemm(dy, w, b_mn=True)
    dw = dyᵀ · x     gemm(dy, x, a_mn=True, b_mn=True)
"""

from __future__ import annotations

import torch

from titan_b200.ops import _lib

__all__ = ["gemm", "linear", "gemm_ref", "supported"]


def gemm_ref(a, b, a_mn=False, b_mn=False, out_dtype=None):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    return (A @ B).to(out_dtype or a.dtype)


def supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    return (_lib.on_device(a) and a.dtype in (torch.bfloat16, torch.float16) and a.dtype == b.dtype
            and a.dim() == 2 and b.dim() == 2)


_POLICY = {"auto": 0, "single": 1, "pair": 2}
_WS: dict = {}


def _workspace(device: torch.device) -> torch.Tensor:
    """Zero-filled partial-sum workspace of the pair kernel's tail split, one per (device, stream): the kernel
    leaves it zeroed, and calls on one stream are ordered, so every GEMM of that stream shares it."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _WS.get(key)
    if ws is None:
        fn = _lib.lib().tb_gemm_ws_bytes
        fn.restype, fn.argtypes = _lib.c_longlong, []
        ws = torch.zeros(int(fn()), dtype=torch.uint8, device=device)
        _WS[key] = ws
    return ws


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None, accumulate: bool = False, max_ctas: int = 0,
         policy: str = "auto", split_tail: bool = True) -> torch.Tensor:
    """A · B.  a: [M,K] (or [K,M] if a_mn); b: [N,K] (or [K,N] if b_mn) → [M,N].

    ``policy``: "auto" picks CTA pairs for problems that fill the GPU, "single" / "pair" force a kernel.
    ``split_tail=False`` keeps the pair kernel's last partial wave as whole tiles (no workspace)."""
    if not supported(a, b):
        raise _lib.KernelError(f"gemm: unsupported operands {a.dtype}{tuple(a.shape)} x {b.dtype}{tuple(b.shape)}")
    if a.stride(-1) != 1:
        a = a.contiguous()
    if b.stride(-1) != 1:
        b = b.contiguous()
    K, M = (a.shape[0], a.shape[1]) if a_mn else (a.shape[1], a.shape[0])
    Kb, N = (b.shape[0], b.shape[1]) if b_mn else (b.shape[1], b.shape[0])
    if K != Kb:
        raise ValueError(f"gemm: contraction mismatch {K} vs {Kb}")
    out_dtype = out_dtype or (out.dtype if out is not None else a.dtype)
    if out_dtype not in (a.dtype, torch.float32):
        raise ValueError("gemm: output dtype must be the input dtype or float32")
    if out is None:
        if accumulate:
            raise ValueError("gemm: accumulate needs an output tensor")
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    elif out.shape != (M, N) or out.stride(-1) != 1:
        raise ValueError("gemm: `out` must be [M, N] with unit inner stride")
    # the kernel needs 16-byte aligned rows: pad ragged leading dimensions through a copy
    if a.stride(0) % 8 or a.data_ptr() % 16:
        a = _aligned_copy(a)
    if b.stride(0) % 8 or b.data_ptr() % 16:
        b = _aligned_copy(b)
    status = _lib.shared_status()
    ws = _workspace(a.device) if split_tail and policy != "single" and a.is_cuda else None
    rc = _lib.lib().tb_gemm_auto(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                                 out.stride(0), int(a_mn), int(b_mn), _lib.dtype_code(a.dtype),
                                 int(out_dtype == torch.float32), int(accumulate), _POLICY[policy],
                                 None if ws is None else ws.data_ptr(), 0 if ws is None else ws.numel(),
                                 int(max_ctas), status.ptr, _lib.stream_ptr())
    _lib.check(rc, "gemm_bf16")
    return out


def _aligned_copy(t: torch.Tensor) -> torch.Tensor:
    rows, cols = t.shape
    ld = (cols + 7) // 8 * 8
    buf = torch.zeros(rows, ld, dtype=t.dtype, device=t.device)
    buf[:, :cols] = t
    return buf[:, :cols]


def _op():
    """The dispatcher ops (`torch.ops.titan_b200`): selective AC, `torch.compile` and meta runs see these."""
    from titan_b200.ops import registry

    return registry.ops


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        y = _op().gemm(x2, w)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        x2 = x.reshape(-1, x.shape[-1])
        g2 = gy.reshape(-1, gy.shape[-1])
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = _op().gemm(g2, w, False, True).view(x.shape)
        if ctx.needs_input_grad[1]:
            dw = _op().gemm(g2, x2, True, True)
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` on the tcgen05 kernel (CUDA bf16/fp16), else `F.linear`."""
    if (x.is_cuda or x.is_meta) and x.dtype in (torch.bfloat16, torch.float16) and w.dtype == x.dtype \
            and x.shape[-1] % 8 == 0 \
            and w.shape[0] % 8 == 0:
        y = _LinearFn.apply(x, w)
        return y if bias is None else y + bias
    return torch.nn.functional.linear(x, w, bias)
