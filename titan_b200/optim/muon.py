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
    returns the update shards; tensor-parallel shards are all-gathered over ``tp`` before that exchange and the
    update is sliced back; under HSDP the exchange stays inside the shard group and the update may be averaged over
    the replicas (``muon_extra_reduce_for_hsdp``);
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

__all__ = ["zeropower_via_newtonschulz5", "normalise_update", "DistributedMuon", "SwapDistributedMuon",
           "split_parameters_for_muon",
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
        if _tc_takes(x):
            x = _ns_step_tc(x, a, b, c)
            continue
        gram = torch.bmm(x, x.transpose(1, 2))
        poly = b * gram + c * torch.bmm(gram, gram)
        x = a * x + torch.bmm(poly, x)
    if transposed:
        x = x.transpose(1, 2)
    return (x.squeeze(0) if two_d else x).to(grad.dtype)


TC_MIN_DIM = 256   # below this a matrix does not fill the tensor-core tiles: the batched library product stays
TC_MAX_BATCH = 16  # one launch per matrix and product: large batches of small experts stay batched


def _tc_takes(x: torch.Tensor) -> bool:
    """x [batch, m, n] (m <= n) contiguous bf16 on a B200 with tile-friendly sizes: the three products of a
    Newton-Schulz step run on the tcgen05 GEMM (`titan_b200.ops.gemm`)."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[0] <= TC_MAX_BATCH and x.shape[1] >= TC_MIN_DIM
            and x.shape[1] % 8 == 0 and x.shape[2] % 8 == 0)


def _ns_step_tc(x: torch.Tensor, a: float, b: float, c: float) -> torch.Tensor:
    """One quintic step X <- aX + (bA + cA^2) X with A = X X^T: no operand is transposed in memory.  A = X X^T is
    `gemm(X, X)` (both K-major), A^2 = `gemm(A, A)` (A is symmetric), and (.) X reads X as the [K, N] operand."""
    from titan_b200.ops.gemm import gemm

    out = torch.empty_like(x)
    for i in range(x.shape[0]):
        xi = x[i].contiguous()
        gram = gemm(xi, xi)
        poly = torch.add(b * gram, gemm(gram, gram), alpha=c)
        out[i] = torch.add(gemm(poly, xi, b_mn=True), xi, alpha=a)
    return out


def normalise_update(u: torch.Tensor, adjust_lr_fn: str | None = "original") -> torch.Tensor:
    a, b = u.size(-2), u.size(-1)
    if adjust_lr_fn in (None, "original"):
        return u * math.sqrt(max(1, a / b))
    if adjust_lr_fn == "match_rms_adamw":
        return u * (0.18 * math.sqrt(max(a, b)))
    raise ValueError(f"unknown muon_adjust_lr_fn {adjust_lr_fn!r}")


def _lmo(g, steps, hybrid, adjust):
    return normalise_update(zeropower_via_newtonschulz5(g, steps=steps, hybrid_ns=hybrid), adjust)


def _all_to_all(recv: list[torch.Tensor], send: list[torch.Tensor], group) -> None:
    """List all-to-all of flat tensors as ONE variable-split `all_to_all_single` (also what gloo offers)."""
    inp = torch.cat([t.reshape(-1) for t in send])
    out = torch.empty(sum(t.numel() for t in recv), dtype=inp.dtype, device=inp.device)
    dist.all_to_all_single(out, inp, output_split_sizes=[t.numel() for t in recv],
                           input_split_sizes=[t.numel() for t in send], group=group)
    o = 0
    for t in recv:
        t.copy_(out[o:o + t.numel()].view(t.shape))
        o += t.numel()


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
                 ns_steps=5, adjust_lr_fn="match_rms_adamw", hybrid_ns=False, dp_group=None,
                 extra_reduce_for_hsdp: bool = False):
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
        self.extra_reduce_for_hsdp = extra_reduce_for_hsdp
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

    # ---- momentum residency (overridden by the swapped variant)
    def _merge_groups(self, params: list) -> list[list]:
        """Parameters are updated group by group; every group's momentum is on the device while it is processed."""
        return [params]

    def _acquire(self, params: list, upcoming: list | None) -> None:
        pass

    def _release(self, params: list) -> None:
        pass

    # ---- step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            active = [p for p in group["params"] if p.grad is not None]
            chunks = self._merge_groups(active)
            for ci, chunk in enumerate(chunks):
                self._acquire(chunk, chunks[ci + 1] if ci + 1 < len(chunks) else None)
                kinds: dict[str, list] = {"expert": [], "fsdp": [], "ddp": [], "local": []}
                for p in chunk:
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
                self._release(chunk)
        return loss

    # ---- how a sharded matrix is laid out over its mesh
    @staticmethod
    def _layout(p: DTensor):
        """→ (fsdp mesh dim | None, tp mesh dim | None, tensor dim split by tp, replicate mesh dim | None).  Mesh axes
        are told apart by name: ``tp`` splits for tensor parallelism, ``dp_replicate*`` replicates (HSDP), every other
        sharding axis is a data-parallel (FSDP) split of dim 0."""
        mesh = p.device_mesh
        names = mesh.mesh_dim_names or tuple(f"dim{i}" for i in range(mesh.ndim))
        fsdp_dim = tp_dim = tp_tensor_dim = rep_dim = None
        for i, (name, pl) in enumerate(zip(names, p.placements)):
            if mesh.size(i) == 1:
                continue
            if isinstance(pl, Shard) or type(pl).__name__ == "_StridedShard":
                if name == "tp":
                    tp_dim, tp_tensor_dim = i, pl.dim
                elif pl.dim == 0 and fsdp_dim is None:
                    fsdp_dim = i
                else:
                    return None
            elif name.startswith("dp_replicate"):
                rep_dim = i
        return fsdp_dim, tp_dim, tp_tensor_dim, rep_dim

    def _step_fsdp(self, items, group) -> None:
        """Buckets of `world` dim-0-sharded matrices: a2a shards → owner orthogonalises → a2a updates back.

        Tensor-parallel shards are all-gathered over ``tp`` first (every tp rank then takes part in the same exchange
        over its own data-parallel group and keeps its slice of the update); under HSDP the exchange runs inside the
        shard group and the update can be averaged over the replicas (``extra_reduce_for_hsdp``) so that they stay
        bit-identical.  When FSDP and TP both split dim 0 the gathered rows arrive in (data rank, tp rank) order
        instead of (tp rank, data rank): Newton-Schulz commutes with row permutations, so nothing is reordered."""
        steps, hyb, adj = group["backend_steps"], group["hybrid_ns"], group["adjust_lr_fn"]
        by_key: dict = {}
        for p, g in items:
            lay = self._layout(p)
            key = (id(p.device_mesh), lay) if lay is not None and lay[0] is not None else None
            by_key.setdefault(key, []).append((p, g))
        for key, lst in by_key.items():
            if key is None:
                # layouts the exchange does not cover: gather, orthogonalise everywhere, keep the local slice
                for p, g in lst:
                    full = g.full_tensor()
                    u = _lmo(full, steps, hyb, adj)
                    self._apply(p, self._slice_like(p, u), group)
                continue
            mesh = lst[0][0].device_mesh
            fsdp_dim, tp_dim, tp_tensor_dim, rep_dim = key[1]
            pg = mesh.get_group(fsdp_dim)
            tp_pg = mesh.get_group(tp_dim) if tp_dim is not None else None
            rep_pg = mesh.get_group(rep_dim) if (rep_dim is not None and self.extra_reduce_for_hsdp) else None
            world, rank = dist.get_world_size(pg), dist.get_rank(pg)
            tp_world = dist.get_world_size(tp_pg) if tp_pg is not None else 1
            tp_rank = dist.get_rank(tp_pg) if tp_pg is not None else 0

            def local_rows(p, g):
                """This data rank's rows of the matrix with the tp split undone."""
                gl = g.to_local().contiguous().bfloat16()
                if tp_pg is None:
                    return gl
                parts = [torch.empty_like(gl) for _ in range(tp_world)]
                dist.all_gather(parts, gl, group=tp_pg)
                self.comm_calls += 1
                return torch.cat(parts, dim=tp_tensor_dim)

            lst = sorted(lst, key=lambda t: t[0].numel(), reverse=True)
            for b0 in range(0, len(lst), world):
                bucket = lst[b0:b0 + world]
                rows_of = [local_rows(p, g) for p, g in bucket]
                dev = rows_of[0].device
                empty = lambda: torch.empty(0, dtype=torch.bfloat16, device=dev)  # noqa: E731
                send = [rows_of[j].reshape(-1) if j < len(bucket) else empty() for j in range(world)]
                if rank < len(bucket):
                    p_own = bucket[rank][0]
                    cols = math.prod(p_own.shape[1:])
                    if tp_pg is None:
                        rows = [self._shard_rows(p_own.shape[0], r, world) for r in range(world)]
                    else:  # even splits only (checked by the DTensor layout of tensor-parallel linears)
                        rows = [p_own.shape[0] // world] * world
                    recv = [torch.empty(rw * cols, dtype=torch.bfloat16, device=dev) for rw in rows]
                else:
                    recv = [empty() for _ in range(world)]
                _all_to_all(recv, send, pg)
                self.comm_calls += 1
                back_send = [empty() for _ in range(world)]
                if rank < len(bucket):
                    p_own = bucket[rank][0]
                    full = torch.cat(recv).view(p_own.shape)
                    u = _lmo(full, steps, hyb, adj).reshape(p_own.shape[0], -1)
                    if rep_pg is not None:
                        dist.all_reduce(u, group=rep_pg, op=dist.ReduceOp.AVG)
                        self.comm_calls += 1
                    r0 = 0
                    for r in range(world):
                        back_send[r] = u[r0:r0 + rows[r]].contiguous().reshape(-1)
                        r0 += rows[r]
                back_recv = [torch.empty(rows_of[j].numel(), dtype=torch.bfloat16, device=dev) if j < len(bucket)
                             else empty() for j in range(world)]
                _all_to_all(back_recv, back_send, pg)
                self.comm_calls += 1
                for j, (p, _) in enumerate(bucket):
                    u_rows = back_recv[j].view(rows_of[j].shape)
                    if tp_pg is not None:
                        u_rows = u_rows.chunk(tp_world, dim=tp_tensor_dim)[tp_rank]
                    self._apply(p, u_rows.reshape(p.to_local().shape), group)

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


class SwapDistributedMuon(DistributedMuon):
    """Muon whose momentum buffers live in pinned host memory between (and during most of) the step.

    All momenta of the optimizer sit in ONE pinned arena in parameter order.  `step()` walks the parameters in
    merge groups of ``swap_merge_buckets`` exchange buckets (``buckets x data-parallel world`` matrices); while one
    group is orthogonalised its momenta are on the device, the next group's are already being copied in on a side
    stream and the previous group's are draining back on another, so at most three groups of momentum are resident.
    On CPU (hardware-free tests) the buffers are plain views of the arena.

    Parity: `SwapMuonState` / the Muon swap hooks of the reference
    (torchtitan_npu/patches/optimizer/swap_optimizer.py:693-1092, muon_optimizer.py:665-753)."""

    def __init__(self, params, names, *, swap_merge_buckets: int = 1, **kw):
        super().__init__(params, names, **kw)
        self.swap_merge_buckets = max(int(swap_merge_buckets), 1)
        self.params_list = [p for g in self.param_groups for p in g["params"]]
        locs = [p.to_local() if isinstance(p, DTensor) else p for p in self.params_list]
        self.offsets = [0]
        for t in locs:
            self.offsets.append(self.offsets[-1] + t.numel())
        self.index = {id(p): i for i, p in enumerate(self.params_list)}
        self.on_cuda = any(t.is_cuda for t in locs)
        dtype = locs[0].dtype if locs else torch.float32
        self.mom_host = torch.zeros(self.offsets[-1], dtype=dtype, pin_memory=self.on_cuda)
        self.h2d_stream = self.d2h_stream = None
        self._inflight: dict[int, tuple] = {}     # id(p) -> (device buffer, "loaded" event) of prefetched momenta
        self._draining: list = []                 # (device buffer, "offloaded" event) kept alive until the copy landed
        self.h2d_bytes = self.d2h_bytes = 0

    def host_view(self, p) -> torch.Tensor:
        i = self.index[id(p)]
        loc = p.to_local() if isinstance(p, DTensor) else p
        return self.mom_host[self.offsets[i]:self.offsets[i + 1]].view(loc.shape)

    def synchronize(self) -> None:
        if self.d2h_stream is not None:
            self.d2h_stream.synchronize()
        self._draining.clear()

    def _merge_groups(self, params: list) -> list[list]:
        world = 1
        for p in params:
            if isinstance(p, DTensor) and p.device_mesh.size() > 1:
                lay = self._layout(p)
                if lay is not None and lay[0] is not None:
                    world = max(world, p.device_mesh.size(lay[0]))
        n = max(self.swap_merge_buckets * world, 1)
        ordered = sorted(params, key=lambda q: q.numel(), reverse=True)   # the exchange buckets are cut in this order
        return [ordered[i:i + n] for i in range(0, len(ordered), n)]

    def _fetch(self, params: list) -> None:
        dev = next(((p.to_local() if isinstance(p, DTensor) else p).device for p in params), None)
        if dev is None or dev.type != "cuda":
            return
        if self.h2d_stream is None:
            self.h2d_stream, self.d2h_stream = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
            self.h2d_stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(self.h2d_stream):
            for p in params:
                if id(p) in self._inflight:
                    continue
                host = self.host_view(p)
                buf = torch.empty(host.shape, dtype=host.dtype, device=dev)
                buf.copy_(host, non_blocking=True)
                self.h2d_bytes += host.numel() * host.element_size()
                ev = torch.cuda.Event()
                ev.record(self.h2d_stream)
                self._inflight[id(p)] = (buf, ev)

    def _acquire(self, params: list, upcoming: list | None) -> None:
        if not self.on_cuda:
            for p in params:
                self.state[p]["momentum_buffer"] = self.host_view(p)
            return
        # the arena may still be receiving the previous step's momenta
        if self.d2h_stream is not None:
            self.h2d_stream.wait_stream(self.d2h_stream)
        self._fetch(params)
        if upcoming:
            self._fetch(upcoming)
        main = torch.cuda.current_stream()
        for p in params:
            buf, ev = self._inflight.pop(id(p))
            main.wait_event(ev)
            buf.record_stream(main)
            self.state[p]["momentum_buffer"] = buf
        self._draining = [(b, e) for b, e in self._draining if not e.query()]

    def _release(self, params: list) -> None:
        if not self.on_cuda:
            for p in params:
                self.state[p].pop("momentum_buffer", None)   # the arena view was updated in place
            return
        main = torch.cuda.current_stream()
        updated = torch.cuda.Event()
        updated.record(main)
        with torch.cuda.stream(self.d2h_stream):
            self.d2h_stream.wait_event(updated)
            for p in params:
                buf = self.state[p].pop("momentum_buffer", None)
                if buf is None:
                    continue
                host = self.host_view(p)
                host.copy_(buf, non_blocking=True)
                self.d2h_bytes += host.numel() * host.element_size()
                ev = torch.cuda.Event()
                ev.record(self.d2h_stream)
                self._draining.append((buf, ev))

    def _effective_grad(self, p, group):
        g = p.grad
        mom = group["momentum"]
        if 0 < mom < 1:
            buf = self.state[p]["momentum_buffer"]
            gl = g.to_local() if isinstance(g, DTensor) else g
            buf.lerp_(gl.to(buf.dtype), 1 - mom)
            out = gl.lerp(buf.to(gl.dtype), mom) if group["nesterov"] else buf
            if isinstance(g, DTensor):
                out = DTensor.from_local(out, g.device_mesh, g.placements, run_check=False, shape=g.shape,
                                         stride=g.stride())
            return out
        return g


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
            muon_kw = dict(lr=muon_lr, momentum=opt_cfg.muon_momentum, nesterov=opt_cfg.muon_enable_nesterov,
                           weight_decay=opt_cfg.weight_decay, ns_steps=opt_cfg.muon_ns_steps,
                           adjust_lr_fn=opt_cfg.muon_adjust_lr_fn, hybrid_ns=opt_cfg.muon_hybrid_ns, dp_group=dp_group,
                           extra_reduce_for_hsdp=getattr(opt_cfg, "muon_extra_reduce_for_hsdp", False))
            if swap:
                self.muon.append(SwapDistributedMuon(groups, names,
                                                     swap_merge_buckets=getattr(opt_cfg, "swap_merge_buckets", 1),
                                                     **muon_kw))
            else:
                self.muon.append(DistributedMuon(groups, names, **muon_kw))
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
        """Flat per-FQN keys.  Swapped halves (AdamW moments, Muon momenta) are emitted from their pinned arenas as
        CPU tensors with the parameter's sharding, under the same keys a resident optimizer writes, so a checkpoint
        taken with swapping loads without it and vice versa."""
        from titan_b200.optim.swap_optimizer import _wrap_like, param_fqns, swap_adamw_state_dict

        opts = StateDictOptions(flatten_optimizer_state_dict=True)
        out: dict[str, Any] = {}
        fqns = param_fqns(self.model_parts)
        for part, mu in zip(self.model_parts, self.muon):
            if isinstance(mu, SwapDistributedMuon):
                mu.synchronize()
                for grp in mu.param_groups:
                    for p in grp["params"]:
                        for fqn in fqns.get(id(p), []):
                            out[f"state.{fqn}.momentum_buffer"] = _wrap_like(p, mu.host_view(p))
                            for k, v in grp.items():
                                if k != "params":
                                    out[f"param_groups.{fqn}.{k}"] = v
            else:
                out.update(get_optimizer_state_dict(part, mu, options=opts))
        for part, ad in zip(self.model_parts, self.adamw):
            if hasattr(ad, "host_views"):
                out.update(swap_adamw_state_dict(ad, fqns))
            else:
                out.update(get_optimizer_state_dict(part, ad, options=opts))
        return out

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        from titan_b200.optim.swap_optimizer import param_fqns, swap_adamw_load_state_dict

        opts = StateDictOptions(flatten_optimizer_state_dict=True)
        fqns = param_fqns(self.model_parts)
        for part, mu in zip(self.model_parts, self.muon):
            if isinstance(mu, SwapDistributedMuon):
                mu.synchronize()
                for grp in mu.param_groups:
                    for p in grp["params"]:
                        fqn = next((f for f in fqns.get(id(p), []) if f"state.{f}.momentum_buffer" in state_dict),
                                   None)
                        if fqn is None:
                            continue
                        src = state_dict[f"state.{fqn}.momentum_buffer"]
                        src = src.to_local() if isinstance(src, DTensor) else src
                        mu.host_view(p).copy_(src.to(mu.mom_host.dtype))
                        for k in list(grp.keys()):
                            if k != "params" and f"param_groups.{fqn}.{k}" in state_dict:
                                grp[k] = state_dict[f"param_groups.{fqn}.{k}"]
            else:
                set_optimizer_state_dict(part, mu, optim_state_dict=state_dict, options=opts)
        swapped = [ad for ad in self.adamw if hasattr(ad, "host_views")]
        if swapped:
            swap_adamw_load_state_dict(swapped, fqns, state_dict)
        for part, ad in zip(self.model_parts, self.adamw):
            if not hasattr(ad, "host_views"):
                # a checkpoint written by the swapped optimizer has no entries for the hyper-parameters that only
                # torch's AdamW knows (maximize, foreach, ...): keep this optimizer's own values for those
                filled = dict(state_dict)
                for grp in ad.param_groups:
                    for p in grp["params"]:
                        for fqn in fqns.get(id(p), []):
                            for k, v in grp.items():
                                if k != "params":
                                    filled.setdefault(f"param_groups.{fqn}.{k}", v)
                set_optimizer_state_dict(part, ad, optim_state_dict=filled, options=opts)

    def init_cache_state_dict(self) -> None:
        for o in [*self.adamw, *self.muon]:
            if hasattr(o, "synchronize"):
                o.synchronize()


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
