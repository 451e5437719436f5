"""AdamW / Adam whose step is ONE multi-tensor sm_100a kernel sequence per dtype group.

Parameters may be plain tensors or DTensors (FSDP2 shards: the kernel updates the local shard;
state is created as DTensors of the same layout so DCP reshards it).  Moments are fp32 (or bf16
with ``state_dtype=torch.bfloat16``).  ``grad_scale`` (a device scalar, e.g. the clip coefficient)
is multiplied into the gradients inside the kernel, so clipping needs no separate pass.

On CPU tensors the same update runs as plain PyTorch math (used by hardware-free tests).

Parity: replaces per-parameter `torch._fused_adamw_` calls (torchtitan_npu/patches/optimizer/
swap_optimizer.py:574-591) with a multi-tensor launch (`csrc/elementwise/adamw.cu`).
"""

from __future__ import annotations

import ctypes
import math

import torch
from torch.distributed.tensor import DTensor
from torch.optim import Optimizer

from titan_b200.ops import _lib

__all__ = ["FusedAdamW", "adamw_multi_tensor", "adamw_reference_step"]


def _local(t):
    return t.to_local() if isinstance(t, DTensor) else t


def adamw_reference_step(p, g, m, v, *, lr, beta1, beta2, eps, wd, step, decoupled=True, grad_scale=1.0,
                         vmax=None, maximize=False):
    """The kernel's arithmetic in PyTorch fp32 (oracle and CPU path); updates in place."""
    pf, gf = p.float(), g.float() * float(grad_scale)
    if maximize:
        gf = -gf
    if decoupled:
        pf = pf - lr * wd * pf
    else:
        gf = gf + wd * pf
    mf = beta1 * m.float() + (1 - beta1) * gf
    vf = beta2 * v.float() + (1 - beta2) * gf * gf
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    dv = vf
    if vmax is not None:
        dv = torch.maximum(vmax.float(), vf)
        vmax.copy_(dv)
    pf = pf - (lr / bc1) * mf / (dv.sqrt() / math.sqrt(bc2) + eps)
    p.copy_(pf)
    m.copy_(mf)
    v.copy_(vf)


def adamw_multi_tensor(params, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs=None, *, lr, beta1, beta2, eps,
                       weight_decay, step, decoupled=True, grad_scale: torch.Tensor | None = None, maximize=False):
    """Launch the fused update on lists of CUDA tensors that share (param, grad, state) dtypes."""
    n = len(params)
    if n == 0:
        return
    amsgrad = max_exp_avg_sqs is not None
    VP = ctypes.c_void_p * n
    arr = lambda ts: VP(*[t.data_ptr() for t in ts])  # noqa: E731
    numel = (ctypes.c_longlong * n)(*[t.numel() for t in params])
    for group in (params, grads, exp_avgs, exp_avg_sqs):
        for t in group:
            if not t.is_contiguous():
                raise _lib.KernelError("fused AdamW needs contiguous tensors")
    rc = _lib.lib().tb_adamw_multi(
        arr(params), arr(grads), arr(exp_avgs), arr(exp_avg_sqs), arr(max_exp_avg_sqs) if amsgrad else None, numel, n,
        float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), int(step), _lib.ptr(grad_scale),
        int(decoupled), int(amsgrad), int(maximize), _lib.dtype_code(params[0].dtype),
        _lib.dtype_code(grads[0].dtype), _lib.dtype_code(exp_avgs[0].dtype), _lib.stream_ptr())
    _lib.check(rc, "adamw_multi")


class FusedAdamW(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, decoupled=True,
                 amsgrad=False, maximize=False, state_dtype=torch.float32):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decoupled=decoupled, amsgrad=amsgrad,
                        maximize=maximize)
        super().__init__(params, defaults)
        self.state_dtype = state_dtype
        self.grad_scale: torch.Tensor | None = None
        self.launches = 0

    def _init_state(self, p):
        st = self.state[p]
        if len(st) == 0:
            st["step"] = torch.tensor(0.0, dtype=torch.float32)
            st["exp_avg"] = torch.zeros_like(p, dtype=self.state_dtype)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=self.state_dtype)
            if self.defaults["amsgrad"]:
                st["max_exp_avg_sq"] = torch.zeros_like(p, dtype=self.state_dtype)
        return st

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            lr = group["lr"]
            lr = float(lr) if not isinstance(lr, torch.Tensor) else float(lr.item())
            buckets: dict = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self._init_state(p)
                st["step"] += 1
                step = int(st["step"].item())
                pl, gl = _local(p), _local(p.grad)
                ml, vl = _local(st["exp_avg"]), _local(st["exp_avg_sq"])
                xl = _local(st["max_exp_avg_sq"]) if group["amsgrad"] else None
                if pl.numel() == 0:
                    continue
                if not pl.is_cuda:
                    gs = float(self.grad_scale) if self.grad_scale is not None else 1.0
                    adamw_reference_step(pl, gl, ml, vl, lr=lr, beta1=beta1, beta2=beta2, eps=group["eps"],
                                         wd=group["weight_decay"], step=step, decoupled=group["decoupled"],
                                         grad_scale=gs, vmax=xl, maximize=group["maximize"])
                    continue
                if not gl.is_contiguous():
                    gl = gl.contiguous()
                key = (step, pl.dtype, gl.dtype, ml.dtype, pl.device)
                b = buckets.setdefault(key, ([], [], [], [], []))
                b[0].append(pl); b[1].append(gl); b[2].append(ml); b[3].append(vl)
                if xl is not None:
                    b[4].append(xl)
            for (step, *_), (ps, gs_, ms, vs, xs) in buckets.items():
                adamw_multi_tensor(ps, gs_, ms, vs, xs if group["amsgrad"] else None, lr=lr, beta1=beta1, beta2=beta2,
                                   eps=group["eps"], weight_decay=group["weight_decay"], step=step,
                                   decoupled=group["decoupled"], grad_scale=self.grad_scale,
                                   maximize=group["maximize"])
                self.launches += 1
        return loss
