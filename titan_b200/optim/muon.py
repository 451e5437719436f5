"""Distributed Muon (+ AdamW for the rest) and the hybrid container / LR schedulers around it.

Parameter split: 2-D matrices (except embeddings, the LM head and ``output``) and 3-D expert stacks go to
Muon; everything else to AdamW.  Muon update of a matrix G (momentum-averaged gradient, optionally Nesterov):

    U = NewtonSchulz(G)            5 quintic iterations in bf16 (or 8 primary + 2 secondary "hybrid" steps)
    U *= sqrt(max(1, A/B))         ("original")   or   0.18 * sqrt(max(A, B))   ("match_rms_adamw")
    p *= 1 - lr * wd ;  p -= lr * U

Routing by how a parameter is distributed:
  * expert stacks (3-D, expert parallel on dim 0, name contains "expert"): every rank orthogonalises its local
    experts, no communication;
  * FSDP-sharded matrices (dim-0 shards): parameters are processed in buckets of `world` matrices; one
    all-to-all gives every rank ONE whole matrix of the bucket, it runs Newton–Schulz, a second all-to-all
    returns the update shards;
  * replicated matrices (DDP / single device): owner-computes with snake-interleaved ownership (largest first)
    and an all-gather of the updates; on one rank this degenerates to a plain local update.

Parity: torchtitan_npu/patches/optimizer/muon_optimizer.py:47-87 (Newton–Schulz), :207-1130 (DistributedMuon),
:1136-1173 (parameter split), :1240-1352 (hybrid container), :1417-1559 (schedulers, warmup-stable-decay).
"""

from __future__ import annotations

import math
import re
from typing import Any

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.checkpoint.state_dict import (
    StateDictOptions,
    get_optimizer_state_dict,
    set_optimizer_state_dict,
)
from torch.distributed.checkpoint.stateful import Stateful
from torch.distributed.tensor import DTensor, Shard
from torch.optim import Optimizer

from titan_b200.utils.logging import logger

__all__ = ["zeropower_via_newtonschulz5", "normalise_update", "DistributedMuon", "split_parameters_for_muon",
           "MuonHybridOptimizersContainer", "build_muon_optimizers", "COEFF_PRIMARY", "COEFF_SECONDARY"]

COEFF_PRIMARY = (3.4445, -4.7750, 2.0315)
COEFF_SECONDARY = (2.0, -1.5, 0.5)  # last two hybrid steps pull singular values exactly to 1
_EXCLUDED = ("tok_embeddings", "embed", "lm_head", "output")
_EXPERT_KEYWORDS = ("experts", "expert")


def zeropower_via_newtonschulz5(grad: torch.Tensor, steps: int = 5, eps: float = 1e-7, hybrid_ns: bool = False):
    """Orthogonalise a matrix (or a batch of matrices) with the quintic Newton–Schulz iteration in bf16."""
    if steps >= 100:
        raise ValueError(f"number of Newton-Schulz steps must be < 100, got {steps}")
    if grad.dim() not in (2, 3):
        raise ValueError(f"Newton-Schulz needs 2-D or 3-D tensors, got shape {tuple(grad.shape)}")
    two_d = grad.dim() == 2
    x = (grad.unsqueeze(0) if two_d else grad).bfloat16()
    transposed = x.shape[-2] > x.shape[-1]
    if transposed:
        x = x.transpose(1, 2)
    x = x / (torch.linalg.norm(x.float(), dim=(-2, -1), keepdim=True).to(x.dtype) + eps)
    a, b, c = COEFF_PRIMARY
    total = 10 if hybrid_ns else steps
    for i in range(total):
        if hybrid_ns and i >= 8:
            a, b, c = COEFF_SECONDARY
        gram = torch.bmm(x, x.transpose(1, 2))
        poly = b * gram + c * torch.bmm(gram, gram)
        x = a * x + torch.bmm(poly, x)
    if transposed:
        x = x.transpose(1, 2)
    return (x.squeeze(0) if two_d else x).to(grad.dtype)


def normalise_update(u: torch.Tensor, adjust_lr_fn: str | None = "original") -> torch.Tensor:
    a, b = u.size(-2), u.size(-1)
    if adjust_lr_fn in (None, "original"):
        return u * math.sqrt(max(1, a / b))
    if adjust_lr_fn == "match_rms_adamw":
        return u * (0.18 * math.sqrt(max(a, b)))
    raise ValueError(f"unknown muon_adjust_lr_fn {adjust_lr_fn!r}")


def _lmo(g, steps, hybrid, adjust):
    return normalise_update(zeropower_via_newtonschulz5(g, steps=steps, hybrid_ns=hybrid), adjust)


def _snake(items: list, w: int) -> list:
    if w <= 1:
        return items
    blocks = [items[i:i + w] for i in range(0, len(items), w)]
    for b, blk in enumerate(blocks):
        if b % 2 == 1:
            blk.reverse()
    return [x for blk in blocks for x in blk]


def _classify(name: str, p) -> str | None:
    if not p.requires_grad:
        return None
    if p.dim() == 2:
        return "adamw" if any(k in name for k in _EXCLUDED) else "muon"
    return "muon" if p.dim() == 3 else "adamw"


def split_parameters_for_muon(model_parts: list[nn.Module]):
    mp, mn, ap, an = [], [], [], []
    for part in model_parts:
        for name, p in part.named_parameters():
            c = _classify(name, p)
            if c == "muon":
                mp.append(p); mn.append(name)
            elif c == "adamw":
                ap.append(p); an.append(name)
    return mp, mn, ap, an


class DistributedMuon(Optimizer):
    def __init__(self, params, names: list[str], *, lr=1e-3, momentum=0.95, nesterov=True, weight_decay=0.0,
                 ns_steps=5, adjust_lr_fn="match_rms_adamw", hybrid_ns=False, dp_group=None):
        if isinstance(params, list) and params and isinstance(params[0], dict):
            groups = params
        else:
            groups = [{"params": list(params)}]
        defaults = dict(lr=lr, momentum=momentum, nesterov=nesterov, weight_decay=weight_decay, backend_steps=ns_steps,
                        adjust_lr_fn=adjust_lr_fn, hybrid_ns=hybrid_ns)
        super().__init__(groups, defaults)
        flat = [p for g in self.param_groups for p in g["params"]]
        self.names = {id(p): n for p, n in zip(flat, names)}
        self.dp_group = dp_group
        self.comm_calls = 0

    # ---- classification
    def _kind(self, p) -> str:
        name = self.names.get(id(p), "")
        if p.dim() == 3 and any(k in name for k in _EXPERT_KEYWORDS):
            if isinstance(p, DTensor):
                for pl in p.placements:
                    if isinstance(pl, Shard) and pl.dim != 0:
                        raise ValueError(f"{name}: expert weights must be sharded on dim 0 for Muon, got {p.placements}")
            return "expert"
        if isinstance(p, DTensor) and any(isinstance(pl, Shard) for pl in p.placements) and p.device_mesh.size() > 1:
            return "fsdp"
        if self.dp_group is not None and dist.is_initialized() and dist.get_world_size(self.dp_group) > 1:
            return "ddp"
        return "local"

    def _effective_grad(self, p, group):
        g = p.grad
        mom = group["momentum"]
        if 0 < mom < 1:
            st = self.state[p]
            if "momentum_buffer" not in st:
                st["momentum_buffer"] = torch.zeros_like(g)
            buf = st["momentum_buffer"]
            buf.lerp_(g, 1 - mom)
            g = g.lerp(buf, mom) if group["nesterov"] else buf
        return g

    @staticmethod
    def _apply(p, u, group):
        lr, wd = group["lr"], group["weight_decay"]
        pl = p.to_local() if isinstance(p, DTensor) else p
        ul = u.to_local() if isinstance(u, DTensor) else u
        if wd:
            pl.mul_(1 - lr * wd)
        pl.add_(ul.to(pl.dtype), alpha=-lr)

    # ---- step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            kinds: dict[str, list] = {"expert": [], "fsdp": [], "ddp": [], "local": []}
            for p in group["params"]:
                if p.grad is None:
                    continue
                kinds[self._kind(p)].append((p, self._effective_grad(p, group)))
            steps, hyb, adj = group["backend_steps"], group["hybrid_ns"], group["adjust_lr_fn"]
            for p, g in kinds["local"] + kinds["expert"]:
                gl = g.to_local() if isinstance(g, DTensor) else g
                if gl.numel() == 0:
                    continue
                self._apply(p, _lmo(gl, steps, hyb, adj), group)
            if kinds["fsdp"]:
                self._step_fsdp(kinds["fsdp"], group)
            if kinds["ddp"]:
                self._step_ddp(kinds["ddp"], group)
        return loss

    def _step_fsdp(self, items, group) -> None:
        """Buckets of `world` dim-0-sharded matrices: a2a shards → owner orthogonalises → a2a updates back."""
        steps, hyb, adj = group["backend_steps"], group["hybrid_ns"], group["adjust_lr_fn"]
        by_mesh: dict = {}
        for p, g in items:
            by_mesh.setdefault(id(p.device_mesh), []).append((p, g))
        for lst in by_mesh.values():
            mesh = lst[0][0].device_mesh
            if mesh.ndim != 1 or not all(isinstance(p.placements[0], Shard) and p.placements[0].dim == 0 for p, _ in lst):
                # uncommon layouts: gather, orthogonalise everywhere, keep the local slice
                for p, g in lst:
                    full = g.full_tensor()
                    u = _lmo(full, steps, hyb, adj)
                    self._apply(p, self._slice_like(p, u), group)
                continue
            pg = mesh.get_group()
            world, rank = dist.get_world_size(pg), dist.get_rank(pg)
            lst.sort(key=lambda t: t[0].numel(), reverse=True)
            for b0 in range(0, len(lst), world):
                bucket = lst[b0:b0 + world]
                send = []
                for j in range(world):  # rank j will own matrix j of the bucket
                    if j < len(bucket):
                        send.append(bucket[j][1].to_local().contiguous().bfloat16().reshape(-1))
                    else:
                        send.append(torch.empty(0, dtype=torch.bfloat16, device=bucket[0][1].to_local().device))
                recv = None
                if rank < len(bucket):
                    p_own = bucket[rank][0]
                    rows = [self._shard_rows(p_own.shape[0], r, world) for r in range(world)]
                    cols = math.prod(p_own.shape[1:])
                    recv = [torch.empty(rw * cols, dtype=torch.bfloat16, device=send[0].device) for rw in rows]
                else:
                    recv = [torch.empty(0, dtype=torch.bfloat16, device=send[0].device) for _ in range(world)]
                dist.all_to_all(recv, send, group=pg)
                self.comm_calls += 1
                back_send = [torch.empty(0, dtype=torch.bfloat16, device=send[0].device) for _ in range(world)]
                if rank < len(bucket):
                    p_own = bucket[rank][0]
                    full = torch.cat(recv).view(p_own.shape)
                    u = _lmo(full, steps, hyb, adj).reshape(p_own.shape[0], -1)
                    r0 = 0
                    for r in range(world):
                        rw = self._shard_rows(p_own.shape[0], r, world)
                        back_send[r] = u[r0:r0 + rw].contiguous().reshape(-1)
                        r0 += rw
                back_recv = []
                for j in range(world):
                    if j < len(bucket):
                        back_recv.append(torch.empty(bucket[j][0].to_local().numel(), dtype=torch.bfloat16,
                                                     device=send[0].device))
                    else:
                        back_recv.append(torch.empty(0, dtype=torch.bfloat16, device=send[0].device))
                dist.all_to_all(back_recv, back_send, group=pg)
                self.comm_calls += 1
                for j, (p, _) in enumerate(bucket):
                    self._apply(p, back_recv[j].view(p.to_local().shape), group)

    @staticmethod
    def _shard_rows(n: int, r: int, world: int) -> int:
        per = -(-n // world)  # DTensor pads the tail: ceil-sized shards, the last ones may be short or empty
        return max(0, min(per, n - r * per))

    @staticmethod
    def _slice_like(p: DTensor, full_update: torch.Tensor) -> torch.Tensor:
        from torch.distributed.tensor import distribute_tensor

        return distribute_tensor(full_update, p.device_mesh, p.placements).to_local()

    def _step_ddp(self, items, group) -> None:
        steps, hyb, adj = group["backend_steps"], group["hybrid_ns"], group["adjust_lr_fn"]
        pg = self.dp_group
        world, rank = dist.get_world_size(pg), dist.get_rank(pg)
        items = sorted(items, key=lambda t: t[0].numel(), reverse=True)
        order = _snake(list(range(len(items))), world)
        owner = {idx: pos % world for pos, idx in enumerate(order)}
        for b0 in range(0, len(order), world):
            blk = order[b0:b0 + world]
            maxn = max(items[i][0].numel() for i in blk)
            mine = torch.zeros(maxn, dtype=torch.bfloat16, device=items[0][0].device)
            for i in blk:
                if owner[i] == rank:
                    p, g = items[i]
                    mine[: p.numel()] = _lmo(g, steps, hyb, adj).reshape(-1).bfloat16()
            gathered = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(gathered, mine, group=pg)
            self.comm_calls += 1
            for i in blk:
                p, _ = items[i]
                self._apply(p, gathered[owner[i]][: p.numel()].view(p.shape), group)


class MuonHybridOptimizersContainer(Optimizer, Stateful):
    """Muon for matrices + AdamW for the rest, one pair per model part."""

    def __init__(self, model_parts, opt_cfg, parallel_dims=None, swap: bool = False):
        self.model_parts = model_parts
        self.muon: list[DistributedMuon] = []
        self.adamw: list[Optimizer] = []
        all_params = []
        dp_group = None
        if parallel_dims is not None and dist.is_initialized() and parallel_dims.dp_replicate_enabled \
                and not parallel_dims.fsdp_enabled:
            dp_group = parallel_dims.get_mesh("dp_replicate").get_group()
        muon_lr = opt_cfg.lr if (opt_cfg.muon_adjust_lr_fn == "match_rms_adamw" or opt_cfg.muon_lr is None) \
            else opt_cfg.muon_lr
        for part in model_parts:
            mp, mn, ap, an = split_parameters_for_muon([part])
            groups, names = _build_param_groups(mp, mn, opt_cfg.extra_param_group_split_rules)
            self.muon.append(DistributedMuon(groups, names, lr=muon_lr, momentum=opt_cfg.muon_momentum,
                                             nesterov=opt_cfg.muon_enable_nesterov, weight_decay=opt_cfg.weight_decay,
                                             ns_steps=opt_cfg.muon_ns_steps, adjust_lr_fn=opt_cfg.muon_adjust_lr_fn,
                                             hybrid_ns=opt_cfg.muon_hybrid_ns, dp_group=dp_group))
            if ap:
                if swap:
                    from titan_b200.optim.swap_optimizer import SwapAdamW

                    self.adamw.append(SwapAdamW(ap, lr=opt_cfg.lr, betas=(opt_cfg.beta1, opt_cfg.beta2),
                                                eps=opt_cfg.eps, weight_decay=opt_cfg.weight_decay,
                                                swap_times=opt_cfg.swap_optimizer_times))
                else:
                    self.adamw.append(torch.optim.AdamW(ap, lr=opt_cfg.lr, betas=(opt_cfg.beta1, opt_cfg.beta2),
                                                        eps=opt_cfg.eps, weight_decay=opt_cfg.weight_decay))
            all_params += mp + ap
            logger.info("[Muon] %d matrices under Muon, %d tensors under AdamW", len(mp), len(ap))
        Optimizer.__init__(self, all_params, {"lr": opt_cfg.lr})
        self.swap = swap
        self.different_lrs = muon_lr != opt_cfg.lr

    def __iter__(self):
        return iter([*self.muon, *self.adamw])

    def __len__(self):
        return len(self.muon) + len(self.adamw)

    def lr_scheduler_targets(self):
        return [*self.muon, *self.adamw]

    def step(self, *a, **k) -> None:
        for o in self:
            o.step(*a, **k)

    def zero_grad(self, *a, **k) -> None:
        for o in self:
            o.zero_grad(*a, **k)

    def state_dict(self) -> dict[str, Any]:
        opts = StateDictOptions(flatten_optimizer_state_dict=True)
        out: dict[str, Any] = {}
        for part, mu in zip(self.model_parts, self.muon):
            out.update(get_optimizer_state_dict(part, mu, options=opts))
        for part, ad in zip(self.model_parts, self.adamw):
            if hasattr(ad, "host_views"):
                continue  # swapped AdamW state is emitted by its own container when used standalone
            out.update(get_optimizer_state_dict(part, ad, options=opts))
        return out

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        opts = StateDictOptions(flatten_optimizer_state_dict=True)
        for part, mu in zip(self.model_parts, self.muon):
            set_optimizer_state_dict(part, mu, optim_state_dict=state_dict, options=opts)
        for part, ad in zip(self.model_parts, self.adamw):
            if not hasattr(ad, "host_views"):
                set_optimizer_state_dict(part, ad, optim_state_dict=state_dict, options=opts)

    def init_cache_state_dict(self) -> None:
        for ad in self.adamw:
            if hasattr(ad, "synchronize"):
                ad.synchronize()


def _build_param_groups(params, names, rules):
    """Per-regex overrides: each rule ``{'str_match': regex, 'lr': …, 'backend_steps': …}`` carves out a group."""
    if not rules:
        return [{"params": list(params)}], list(names)
    groups: list[dict] = []
    ordered_names: list[str] = []
    taken: set[int] = set()
    for rule in rules:
        rx = re.compile(rule["str_match"])
        sel = [(p, n) for p, n in zip(params, names) if id(p) not in taken and rx.search(n)]
        if not sel:
            continue
        taken.update(id(p) for p, _ in sel)
        g = {"params": [p for p, _ in sel]}
        g.update({k: v for k, v in rule.items() if k != "str_match"})
        groups.append(g)
        ordered_names += [n for _, n in sel]
    rest = [(p, n) for p, n in zip(params, names) if id(p) not in taken]
    if rest:
        groups.append({"params": [p for p, _ in rest]})
        ordered_names += [n for _, n in rest]
    return groups, ordered_names


def build_muon_optimizers(model_parts, opt_cfg, parallel_dims=None, swap: bool = False):
    return MuonHybridOptimizersContainer(model_parts, opt_cfg, parallel_dims, swap=swap)
