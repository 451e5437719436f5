"""Swap Optimizer: AdamW / Adam whose moments live in pinned host memory.

Between steps the device holds parameters and gradients only.  `step()` streams the state through
the GPU in `swap_optimizer_times` slices on three lanes:

    load lane    (side stream)  pinned host ──cudaMemcpyAsync──► device staging slot
    compute lane (main stream)  multi-tensor fused AdamW on the slot (one launch sequence per slice)
    offload lane (side stream)  device staging slot ──cudaMemcpyAsync──► pinned host

Design points that differ from a per-parameter swap: all moments of one optimizer sit in ONE pinned arena
in parameter order, so a slice is a contiguous range and moves with two large DMA transfers (m and v)
instead of two per parameter; two staging slots alternate, so slice s+1 loads while slice s updates and
slice s-1 drains; a slot is reloaded only after its previous offload has finished (event dependency).
Peak extra device memory is ``2 slots · 2 moments · slice_numel · 4 B``.

Checkpointing: `state_dict()` first waits for the offload lane, then emits flat per-FQN keys
(``state.<fqn>.exp_avg``, ``state.<fqn>.exp_avg_sq``, ``state.<fqn>.step``, ``param_groups.<fqn>.<key>``) whose
tensors are views of the pinned arena, re-wrapped as CPU DTensors with the parameter's mesh and placements:
nothing bounces through the GPU and the layout equals that of a resident optimizer, so checkpoints are
interchangeable.  `load_state_dict()` is transactional: on any error the previous state is restored.

Parity: torchtitan_npu/patches/optimizer/swap_optimizer.py:112-674 (three-lane pipeline of
docs/assets/swap_optimizer.png, flat DCP keys :365-434, transactional load :546-556, aliased params by FQN list).
"""

from __future__ import annotations

import copy
from typing import Any

import torch
import torch.nn as nn
from torch.distributed.checkpoint.stateful import Stateful
from torch.distributed.tensor import DTensor
from torch.optim import Optimizer

from titan_b200.optim.fused_adamw import adamw_multi_tensor, adamw_reference_step
from titan_b200.utils.logging import logger

__all__ = ["SwapOptimizersContainer", "SwapAdamW", "param_fqns", "swap_adamw_state_dict",
           "swap_adamw_load_state_dict"]

_PREFIXES = ("_checkpoint_wrapped_module.", "_orig_mod.", "module.")


def _clean(name: str) -> str:
    for p in _PREFIXES:
        name = name.replace(p, "")
    return name


def param_fqns(model_parts: list[nn.Module]) -> dict[int, list[str]]:
    """id(param) → every FQN under which it is reachable (tied parameters have several)."""
    out: dict[int, list[str]] = {}
    for part in model_parts:
        for name, p in part.named_parameters(remove_duplicate=False):
            out.setdefault(id(p), []).append(_clean(name))
    return out


def _local(t):
    return t.to_local() if isinstance(t, DTensor) else t


class SwapAdamW(Optimizer):
    """One optimizer (one model part).  State: pinned arenas `m`, `v` (+ `vmax`) and a host step counter."""

    def __init__(self, params, *, lr, betas, eps, weight_decay, decoupled=True, amsgrad=False, swap_times=16,
                 pin_memory: bool | None = None):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decoupled=decoupled, amsgrad=amsgrad)
        super().__init__(params, defaults)
        self.swap_times = max(int(swap_times), 1)
        self.params_list = [p for g in self.param_groups for p in g["params"]]
        self.group_of = {id(p): g for g in self.param_groups for p in g["params"]}
        numels = [_local(p).numel() for p in self.params_list]
        self.offsets = [0]
        for n in numels:
            self.offsets.append(self.offsets[-1] + n)
        total = self.offsets[-1]
        self.on_cuda = total > 0 and any(_local(p).is_cuda for p in self.params_list)
        pin = self.on_cuda if pin_memory is None else pin_memory
        mk = lambda: torch.zeros(total, dtype=torch.float32, pin_memory=pin)  # noqa: E731
        self.m_host, self.v_host = mk(), mk()
        self.vmax_host = mk() if amsgrad else None
        self.steps = {id(p): 0 for p in self.params_list}
        # slices end at parameter boundaries; target numel per slice = total / swap_times
        target = max(total // self.swap_times, 1)
        self.slices: list[tuple[int, int]] = []
        start, acc = 0, 0
        for i, n in enumerate(numels):
            acc += n
            if acc >= target or i == len(numels) - 1:
                self.slices.append((start, i + 1))
                start, acc = i + 1, 0
        self.slot_numel = max((self.offsets[b] - self.offsets[a] for a, b in self.slices), default=0)
        self._slots = None
        self.h2d_stream = self.d2h_stream = None
        self.launches = 0
        self.grad_scale: torch.Tensor | None = None
        logger.info("[SwapOptimizer] %d params, %d elements, %d slices, slot %.1f MiB x2 x%d", len(numels), total,
                    len(self.slices), self.slot_numel * 4 / 2 ** 20, 3 if amsgrad else 2)

    # ---- device staging (allocated lazily, freed by `release_staging`)
    def _ensure_staging(self, device):
        if self._slots is None:
            n_buf = 3 if self.defaults["amsgrad"] else 2
            self._slots = [[torch.empty(self.slot_numel, dtype=torch.float32, device=device) for _ in range(n_buf)]
                           for _ in range(2)]
            self.h2d_stream, self.d2h_stream = torch.cuda.Stream(device), torch.cuda.Stream(device)
        return self._slots

    def release_staging(self) -> None:
        self.synchronize()
        self._slots = None

    def synchronize(self) -> None:
        if self.d2h_stream is not None:
            self.d2h_stream.synchronize()

    def host_views(self, p) -> dict[str, torch.Tensor]:
        i = next(k for k, q in enumerate(self.params_list) if q is p)
        a, b = self.offsets[i], self.offsets[i + 1]
        shape = _local(p).shape
        out = {"exp_avg": self.m_host[a:b].view(shape), "exp_avg_sq": self.v_host[a:b].view(shape)}
        if self.vmax_host is not None:
            out["max_exp_avg_sq"] = self.vmax_host[a:b].view(shape)
        return out

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if not self.on_cuda:
            self._step_host()
            return loss
        device = next(_local(p).device for p in self.params_list if _local(p).is_cuda)
        slots = self._ensure_staging(device)
        main = torch.cuda.current_stream(device)
        hosts = [self.m_host, self.v_host] + ([self.vmax_host] if self.vmax_host is not None else [])
        d2h_done: list[torch.cuda.Event | None] = [None, None]
        # the arenas may still be draining from the previous step
        self.h2d_stream.wait_stream(self.d2h_stream)
        for s, (pa, pb) in enumerate(self.slices):
            slot = slots[s & 1]
            lo, hi = self.offsets[pa], self.offsets[pb]
            n = hi - lo
            with torch.cuda.stream(self.h2d_stream):
                if d2h_done[s & 1] is not None:
                    self.h2d_stream.wait_event(d2h_done[s & 1])  # the slot's previous contents are safely on the host
                for dev_buf, host in zip(slot, hosts):
                    dev_buf[:n].copy_(host[lo:hi], non_blocking=True)
                loaded = torch.cuda.Event()
                loaded.record(self.h2d_stream)
            main.wait_event(loaded)
            self._update_slice(pa, pb, slot, lo)
            updated = torch.cuda.Event()
            updated.record(main)
            with torch.cuda.stream(self.d2h_stream):
                self.d2h_stream.wait_event(updated)
                for dev_buf, host in zip(slot, hosts):
                    host[lo:hi].copy_(dev_buf[:n], non_blocking=True)
                done = torch.cuda.Event()
                done.record(self.d2h_stream)
            d2h_done[s & 1] = done
        # the next forward may not start overwriting gradients/params the offload lane does not touch: no wait
        return loss

    def _update_slice(self, pa: int, pb: int, slot, lo: int) -> None:
        buckets: dict = {}
        for i in range(pa, pb):
            p = self.params_list[i]
            if p.grad is None:
                continue
            g = self.group_of[id(p)]
            self.steps[id(p)] += 1
            pl, gl = _local(p), _local(p.grad)
            if pl.numel() == 0:
                continue
            if not gl.is_contiguous():
                gl = gl.contiguous()
            a, b = self.offsets[i] - lo, self.offsets[i + 1] - lo
            views = [buf[a:b] for buf in slot]
            key = (id(g), self.steps[id(p)], pl.dtype, gl.dtype)
            bk = buckets.setdefault(key, (g, [], [], [], [], []))
            bk[1].append(pl.reshape(-1) if pl.is_contiguous() else pl)
            bk[2].append(gl.reshape(-1))
            bk[3].append(views[0]); bk[4].append(views[1])
            if len(views) > 2:
                bk[5].append(views[2])
        for (_, step, _, _), (g, ps, gs, ms, vs, xs) in buckets.items():
            lr = g["lr"]
            adamw_multi_tensor(ps, gs, ms, vs, xs if g["amsgrad"] else None, lr=float(lr), beta1=g["betas"][0],
                               beta2=g["betas"][1], eps=g["eps"], weight_decay=g["weight_decay"], step=step,
                               decoupled=g["decoupled"], grad_scale=self.grad_scale)
            self.launches += 1

    def _step_host(self) -> None:
        """CPU parameters (hardware-free tests): same arithmetic, no streams."""
        for i, p in enumerate(self.params_list):
            if p.grad is None:
                continue
            g = self.group_of[id(p)]
            self.steps[id(p)] += 1
            a, b = self.offsets[i], self.offsets[i + 1]
            pl = _local(p)
            shape = pl.shape
            adamw_reference_step(pl, _local(p.grad), self.m_host[a:b].view(shape), self.v_host[a:b].view(shape),
                                 lr=float(g["lr"]), beta1=g["betas"][0], beta2=g["betas"][1], eps=g["eps"],
                                 wd=g["weight_decay"], step=self.steps[id(p)], decoupled=g["decoupled"],
                                 vmax=self.vmax_host[a:b].view(shape) if self.vmax_host is not None else None)


def _wrap_like(p, host_view: torch.Tensor):
    if isinstance(p, DTensor):
        return DTensor.from_local(host_view, p.device_mesh, p.placements, run_check=False, shape=p.shape,
                                  stride=p.stride())
    return host_view


def swap_adamw_state_dict(o: "SwapAdamW", fqns: dict[int, list[str]]) -> dict[str, Any]:
    """Flat checkpoint keys of one swapped optimizer; the tensors are views of its pinned arenas."""
    o.synchronize()
    out: dict[str, Any] = {}
    for p in o.params_list:
        views = o.host_views(p)
        g = o.group_of[id(p)]
        for fqn in fqns.get(id(p), []):
            for k, v in views.items():
                out[f"state.{fqn}.{k}"] = _wrap_like(p, v)
            out[f"state.{fqn}.step"] = torch.tensor(float(o.steps[id(p)]))
            for k, v in g.items():
                if k != "params":
                    out[f"param_groups.{fqn}.{k}"] = (v.detach().cpu().clone() if torch.is_tensor(v)
                                                      else copy.deepcopy(v))
    return out


class SwapOptimizersContainer(Optimizer, Stateful):
    state_keys = ("exp_avg", "exp_avg_sq", "max_exp_avg_sq")

    def __init__(self, model_parts: list[nn.Module], opt_cfg):
        self.model_parts = model_parts
        self.optimizers: list[SwapAdamW] = []
        all_params = []
        kw = dict(lr=opt_cfg.lr, betas=(opt_cfg.beta1, opt_cfg.beta2), eps=opt_cfg.eps,
                  weight_decay=opt_cfg.weight_decay, decoupled=(opt_cfg.name == "AdamW"),
                  swap_times=opt_cfg.swap_optimizer_times)
        for part in model_parts:
            params = [p for p in part.parameters() if p.requires_grad]
            self.optimizers.append(SwapAdamW(params, **kw))
            all_params.extend(params)
        Optimizer.__init__(self, all_params, {"lr": opt_cfg.lr})
        self.fqns = param_fqns(model_parts)

    def __iter__(self):
        return iter(self.optimizers)

    def __len__(self):
        return len(self.optimizers)

    def step(self, *a, **k) -> None:
        for o in self.optimizers:
            o.step(*a, **k)

    def zero_grad(self, *a, **k) -> None:
        for o in self.optimizers:
            o.zero_grad(*a, **k)

    def synchronize(self) -> None:
        for o in self.optimizers:
            o.synchronize()

    def init_cache_state_dict(self) -> None:
        self.synchronize()

    # ---- checkpoint
    _wrap_like = staticmethod(_wrap_like)

    def state_dict(self) -> dict[str, Any]:
        self.synchronize()  # the offload lane owns the arenas until its copies land
        out: dict[str, Any] = {}
        for o in self.optimizers:
            out.update(swap_adamw_state_dict(o, self.fqns))
        return out

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self.synchronize()
        swap_adamw_load_state_dict(self.optimizers, self.fqns, state_dict)
        if torch.cuda.is_available():
            torch.cuda.empty_cache()


def swap_adamw_load_state_dict(optimizers: list["SwapAdamW"], fqns_of: dict[int, list[str]],
                               state_dict: dict[str, Any]) -> None:
    """Transactional load into the pinned arenas of ``optimizers``: on any error the previous state is restored."""
    for o in optimizers:
        o.synchronize()
    backup = [(o, o.m_host.clone(), o.v_host.clone(), None if o.vmax_host is None else o.vmax_host.clone(),
               dict(o.steps), [dict(g) for g in o.param_groups]) for o in optimizers]
    try:
        for o in optimizers:
            for p in o.params_list:
                fqns = fqns_of.get(id(p), [])
                fqn = next((f for f in fqns if f"state.{f}.exp_avg" in state_dict), None)
                if fqn is None:
                    continue
                views = o.host_views(p)
                for k, dst in views.items():
                    src = state_dict.get(f"state.{fqn}.{k}")
                    if src is None:
                        if k == "max_exp_avg_sq":
                            continue
                        raise KeyError(f"state.{fqn}.{k} missing from the optimizer checkpoint")
                    src = _local(src)
                    if tuple(src.shape) != tuple(dst.shape):
                        raise ValueError(f"state.{fqn}.{k}: shape {tuple(src.shape)} != {tuple(dst.shape)}")
                    dst.copy_(src.to(torch.float32))
                st = state_dict.get(f"state.{fqn}.step")
                if st is not None:
                    o.steps[id(p)] = int(float(st))
                g = o.group_of[id(p)]
                for k in list(g.keys()):
                    key = f"param_groups.{fqn}.{k}"
                    if k != "params" and key in state_dict:
                        g[k] = state_dict[key]
    except Exception:
        for o, m, v, x, steps, groups in backup:
            o.m_host.copy_(m); o.v_host.copy_(v)
            if x is not None:
                o.vmax_host.copy_(x)
            o.steps = steps
            for g, old in zip(o.param_groups, groups):
                params = g["params"]
                g.clear(); g.update(old); g["params"] = params
        raise
