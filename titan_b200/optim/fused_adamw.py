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
                       weight_decay, step, decoupled=True, grad_scale: torch.Tensor | None = None, maximize=False,
                       dyn: torch.Tensor | None = None):
    """Launch the fused update on lists of CUDA tensors that share (param, grad, state) dtypes.  ``dyn`` (3 fp32 on
    the device: lr, 1 - beta1^step, 1 / sqrt(1 - beta2^step)) replaces ``lr`` / ``step``: the form a CUDA graph
    records."""
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
    if dyn is not None:
        _declare_dyn()
        rc = _lib.lib().tb_adamw_multi_dyn(
            arr(params), arr(grads), arr(exp_avgs), arr(exp_avg_sqs), arr(max_exp_avg_sqs) if amsgrad else None, numel,
            n, dyn.data_ptr(), float(beta1), float(beta2), float(eps), float(weight_decay), _lib.ptr(grad_scale),
            int(decoupled), int(amsgrad), int(maximize), _lib.dtype_code(params[0].dtype),
            _lib.dtype_code(grads[0].dtype), _lib.dtype_code(exp_avgs[0].dtype), _lib.stream_ptr())
        _lib.check(rc, "adamw_multi_dyn")
        return
    rc = _lib.lib().tb_adamw_multi(
        arr(params), arr(grads), arr(exp_avgs), arr(exp_avg_sqs), arr(max_exp_avg_sqs) if amsgrad else None, numel, n,
        float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), int(step), _lib.ptr(grad_scale),
        int(decoupled), int(amsgrad), int(maximize), _lib.dtype_code(params[0].dtype),
        _lib.dtype_code(grads[0].dtype), _lib.dtype_code(exp_avgs[0].dtype), _lib.stream_ptr())
    _lib.check(rc, "adamw_multi")


_DYN_DECLARED = False


def _declare_dyn() -> None:
    global _DYN_DECLARED
    if not _DYN_DECLARED:
        P, I, LL, Fl = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        _lib.declare("tb_adamw_multi_dyn", [P, P, P, P, P, P, I, P, Fl, Fl, Fl, Fl, P, I, I, I, I, I, I, P])
        _lib.declare("tb_adamw_bias_corrections", [Fl, Fl, LL, P])
        _DYN_DECLARED = True


class FusedAdamW(Optimizer):
    MAX_GRAPHS = 4   # recordings kept in the CUDA-graph form of the step

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, decoupled=True,
                 amsgrad=False, maximize=False, state_dtype=torch.float32, cuda_graph: bool = False):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decoupled=decoupled, amsgrad=amsgrad,
                        maximize=maximize)
        super().__init__(params, defaults)
        self.state_dtype = state_dtype
        self.grad_scale: torch.Tensor | None = None
        self.launches = 0
        # ``cuda_graph``: the whole step (every bucket of every group) is recorded once as a CUDA graph and replayed;
        # the scalars that change per step travel through a small device buffer.  The recording is keyed on the
        # addresses of parameters, gradients and moments (gradients are new tensors each step, but the caching
        # allocator hands back the same blocks in steady state, often alternating between two sets); a few recordings
        # are kept, and an unseen set of addresses is recorded anew.
        self.cuda_graph = cuda_graph
        self._graphs: dict = {}          # address signature -> (graph, scalar buffer, clip-coefficient buffer)
        self.graph_captures = 0
        self.graph_replays = 0

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
        all_buckets = []
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
            all_buckets.append((group, lr, buckets))
        if self.cuda_graph and all_buckets and self._graph_ok(all_buckets):
            self._graph_step(all_buckets)
            return loss
        for group, lr, buckets in all_buckets:
            beta1, beta2 = group["betas"]
            for (step, *_), (ps, gs_, ms, vs, xs) in buckets.items():
                adamw_multi_tensor(ps, gs_, ms, vs, xs if group["amsgrad"] else None, lr=lr, beta1=beta1, beta2=beta2,
                                   eps=group["eps"], weight_decay=group["weight_decay"], step=step,
                                   decoupled=group["decoupled"], grad_scale=self.grad_scale,
                                   maximize=group["maximize"])
                self.launches += 1
        return loss

    def zero_grad(self, set_to_none: bool = True) -> None:
        # a recorded step addresses the gradients it saw: keep them in place (zeroed, then accumulated into) instead
        # of freeing them, or their addresses move every step and every step records anew
        super().zero_grad(set_to_none=set_to_none and not self.cuda_graph)

    # ---- CUDA-graph form of the step
    @staticmethod
    def _graph_ok(all_buckets) -> bool:
        return all(t.is_cuda for _, _, buckets in all_buckets for lists in buckets.values() for t in lists[0])

    def _graph_step(self, all_buckets) -> None:
        flat = [(group, lr, key, lists) for group, lr, buckets in all_buckets for key, lists in buckets.items()]
        sig = tuple((key[1:], tuple(t.data_ptr() for lst in lists for t in lst),
                     group["betas"], group["eps"], group["weight_decay"], group["decoupled"], group["amsgrad"],
                     group["maximize"]) for group, _, key, lists in flat) + (self.grad_scale is not None,)
        dev = flat[0][3][0][0].device
        host = torch.empty(len(flat), 3, dtype=torch.float32, pin_memory=True)
        _declare_dyn()
        bc = (ctypes.c_float * 2)()
        for i, (group, lr, key, _) in enumerate(flat):
            beta1, beta2 = group["betas"]
            _lib.check(_lib.lib().tb_adamw_bias_corrections(float(beta1), float(beta2), int(key[0]), bc), "adamw_bc")
            host[i, 0], host[i, 1], host[i, 2] = lr, bc[0], bc[1]
        entry = self._graphs.get(sig)
        if entry is None:
            dyn = torch.empty(len(flat), 3, dtype=torch.float32, device=dev)
            scale = torch.ones((), dtype=torch.float32, device=dev) if self.grad_scale is not None else None
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i, (group, _, _, (ps, gs_, ms, vs, xs)) in enumerate(flat):
                    beta1, beta2 = group["betas"]
                    adamw_multi_tensor(ps, gs_, ms, vs, xs if group["amsgrad"] else None, lr=0.0, beta1=beta1,
                                       beta2=beta2, eps=group["eps"], weight_decay=group["weight_decay"], step=1,
                                       decoupled=group["decoupled"], grad_scale=scale, maximize=group["maximize"],
                                       dyn=dyn[i])
            if len(self._graphs) >= self.MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))   # oldest recording
            entry = self._graphs[sig] = (graph, dyn, scale)
            self.graph_captures += 1
            from titan_b200.utils.logging import logger

            logger.info("fused AdamW: recorded the step as a CUDA graph (%d launches; recording %d after %d replays)",
                        len(flat), self.graph_captures, self.graph_replays)
            # recording does not execute: the replay below is this step's update
        graph, dyn, scale = entry
        dyn.copy_(host, non_blocking=True)
        if scale is not None:
            scale.copy_(self.grad_scale.reshape(()).float())
        graph.replay()
        self.graph_replays += 1
        self.launches += len(flat)
