"""Meta-device memory and communication simulator: per-rank HBM of a recipe without any GPU.

The model named by a `TrainerConfig` is built on the **meta** device and converted exactly as the
trainer would; one forward + backward of a local batch then runs on meta tensors under
`MetaMemoryTracker`, a dispatch mode that follows every tensor storage created by an operator until
it is freed — the peak of that curve is the activation footprint under the chosen activation-
checkpoint mode.  Static terms (parameter, gradient and optimizer shards, FSDP all-gather /
reduce-scatter buffers) follow from `ParallelDims` arithmetic:

    params    Σ numel / shard(p) · store bytes          shard = fsdp·tp (dense), efsdp·ep·etp (experts), / pp
    optim     2 moments · local params: fp32 with the framework's fused AdamW, the storage dtype with the library
              implementations; 0 on the device with Swap/Virtual optimizers
    gathered  FSDP only: unsharded compute copies that stay resident: every unit with
              ``fsdp_reshard_after_forward = never``, two units (current + prefetched) otherwise
    fsdp buf  all-gather output of the next unit + the gradient bucket of one unit (wire dtype of the chosen
              reduce-scatter) + the unit's unsharded gradients while they wait for the reduction
    dynamic   peak over the forward + backward TIMELINE of (live activations + gradients created so far); a
              gradient counts in full while its layer is in backward and as its 1 / fsdp shard once reduced.
              Activation bytes are divided by tp · cp (sequence- and context-parallel shards).

The peak of a step is NOT activations + gradients: gradients appear while activations are being freed, so on one
GPU an 8B model peaks at the START of backward (weights + optimizer state + all activations, no gradient yet).

The estimate is checked against the HBM budget (180 GB by default) and reports link traffic per
step with the time it costs at NVLink bandwidth.  The fake-backend dry run (`--comm.mode
fake_backend`) executes the real trainer for one step in one process and complements this static
estimate.

The reference has no simulator module; it documents estimation formulas and a snapshot analyser
(.agents/skills/oom-analysis/references/memory-estimation-templates.md:7-107) and a fake-backend
dry run (scripts/run_train.sh:23-27).  This module turns those into a first-class component.
"""

from __future__ import annotations

import json
import weakref
from dataclasses import asdict, dataclass, field

import torch
from torch.utils._python_dispatch import TorchDispatchMode
from torch.utils._pytree import tree_flatten

__all__ = ["MetaMemoryTracker", "MemoryReport", "estimate", "run_from_config"]

GIB = 1024 ** 3


def _meta_bincount(x, weights=None, minlength=0):
    return torch.empty(max(int(minlength), 1), dtype=torch.int64 if weights is None else weights.dtype, device=x.device)


def _meta_histc(x, bins=100, min=0, max=0):
    return torch.empty(int(bins), dtype=x.dtype, device=x.device)


def _meta_nonzero(x):
    return torch.empty(x.numel(), x.dim(), dtype=torch.int64, device=x.device)   # upper bound: every element


# Operators whose output shape depends on values have no meta kernel; the tracker only needs shapes, and for these
# the shape (or a safe upper bound of it) follows from the arguments.
def _meta_masked_select(x, mask):
    shape = torch.broadcast_shapes(x.shape, mask.shape)
    n = 1
    for d in shape:
        n *= d
    return torch.empty(n, dtype=x.dtype, device=x.device)   # upper bound: every element selected


_META_STAND_INS = {
    torch.ops.aten.bincount.default: _meta_bincount,
    torch.ops.aten.histc.default: _meta_histc,
    torch.ops.aten.nonzero.default: _meta_nonzero,
    torch.ops.aten.masked_select.default: _meta_masked_select,
}


class MetaMemoryTracker(TorchDispatchMode):
    """Tracks live bytes of storages created while the mode is active (works on meta tensors)."""

    def __init__(self, cost=None):
        super().__init__()
        self.current = 0
        self.peak = 0
        self._seen: dict[int, int] = {}
        self.cost = cost   # optional `simulator.cost.StepCost`: prices every operator that passes through

    def _release(self, key: int) -> None:
        self.current -= self._seen.pop(key, 0)

    def _track(self, t: torch.Tensor) -> None:
        try:
            st = t.untyped_storage()
        except Exception:
            return
        key = id(st)
        if key in self._seen:
            return
        n = st.nbytes()
        if n == 0:
            n = t.numel() * t.element_size()
        self._seen[key] = n
        self.current += n
        self.peak = max(self.peak, self.current)
        weakref.finalize(st, self._release, key)

    def reweight(self, t: torch.Tensor, factor: float) -> None:
        """Count the storage of ``t`` as ``factor`` of its size from now on (a gradient that has been reduce-scattered
        keeps 1 / fsdp of its bytes on this rank)."""
        try:
            key = id(t.untyped_storage())
        except Exception:
            return
        n = self._seen.get(key)
        if n is None:
            return
        new = int(n * factor)
        self._seen[key] = new
        self.current -= n - new

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        try:
            out = func(*args, **(kwargs or {}))
        except NotImplementedError:
            stand_in = _META_STAND_INS.get(func)
            if stand_in is None:
                raise
            out = stand_in(*args, **(kwargs or {}))
        if self.cost is not None:
            try:
                self.cost.on_op(func, args, kwargs or {}, out)
            except Exception:   # pricing an operator must never break the memory estimate
                self.cost.unpriced += 1
        # storages that came IN with the arguments are not allocations of this op: a view of a parameter (``w.t()``)
        # shares the parameter's storage, which the static terms already count
        for leaf in tree_flatten((args, kwargs or {}))[0]:
            if isinstance(leaf, torch.Tensor):
                try:
                    key = id(leaf.untyped_storage())
                except Exception:
                    continue
                if key not in self._seen:
                    self._seen[key] = 0
                    weakref.finalize(leaf.untyped_storage(), self._release, key)
        for leaf in tree_flatten(out)[0]:
            if isinstance(leaf, torch.Tensor):
                self._track(leaf)
        return out


@dataclass
class MemoryReport:
    world_size: int
    parallelism: dict
    params_total: int
    params_local: int
    bytes_params: int
    bytes_grads: int
    bytes_optimizer_device: int
    bytes_optimizer_host: int
    bytes_fsdp_buffers: int
    bytes_activations: int
    bytes_total: int
    budget_bytes: int
    fits: bool
    comm_bytes_per_step: dict = field(default_factory=dict)
    comm_seconds_per_step: float = 0.0
    notes: list = field(default_factory=list)
    bytes_gathered_params: int = 0
    bytes_dynamic_peak: int = 0
    bytes_grads_at_peak: int = 0
    step_seconds_estimate: float = 0.0       # 0 when the step could not be traced
    tokens_per_second_estimate: float = 0.0  # whole job
    flops_per_rank_step: float = 0.0
    seconds_by_kind: dict = field(default_factory=dict)
    operators_per_step: int = 0              # dispatched operators + library launches of the traced step

    def summary(self) -> str:
        g = lambda b: f"{b / GIB:8.2f} GiB"  # noqa: E731
        lines = [
            f"memory estimate per rank ({self.world_size} ranks, {self.parallelism})",
            f"  parameters        {g(self.bytes_params)}   ({self.params_local:,} of {self.params_total:,} params)",
            f"  gradients         {g(self.bytes_grads)}   (at the end of backward; {g(self.bytes_grads_at_peak)} at the peak)",
            f"  optimizer (HBM)   {g(self.bytes_optimizer_device)}   (+{g(self.bytes_optimizer_host)} pinned host)",
            f"  FSDP buffers      {g(self.bytes_fsdp_buffers)}   (+{g(self.bytes_gathered_params)} gathered weights kept)",
            f"  activations       {g(self.bytes_activations)}   (live at the peak of the forward + backward timeline)",
            f"  total             {g(self.bytes_total)}   budget {g(self.budget_bytes)}   "
            f"{'FITS' if self.fits else 'DOES NOT FIT'}",
            f"  link traffic/step {json.dumps({k: round(v / GIB, 3) for k, v in self.comm_bytes_per_step.items()})} GiB"
            f" ≈ {self.comm_seconds_per_step * 1e3:.1f} ms at link rate",
        ]
        if self.step_seconds_estimate > 0:
            top = ", ".join(f"{k} {v * 1e3:.0f} ms" for k, v in list(self.seconds_by_kind.items())[:6])
            lines.append(f"  step time (est.)  {self.step_seconds_estimate * 1e3:8.1f} ms   "
                         f"{self.tokens_per_second_estimate:,.0f} tokens/s for the job   "
                         f"{self.flops_per_rank_step / 1e12:.0f} TFLOP per rank   ({top})")
        return "\n".join(lines + [f"  note: {n}" for n in self.notes])

    def to_json(self) -> str:
        return json.dumps(asdict(self))


_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def _is_expert(name: str) -> bool:
    return ".experts." in name and "shared_experts" not in name


_ACTIVE_COST: list = [None]   # the step-cost model of the run in progress (the attention stand-in reports to it)


class _FlashStandIn(torch.autograd.Function):
    """Memory-faithful stand-in for fused attention on meta tensors: keeps q, k, v, out and the
    log-sum-exp row statistics alive for backward and never materialises the score matrix (the math
    fallback that meta tensors would otherwise take allocates [B, H, S, S])."""

    @staticmethod
    def forward(ctx, q, k, v):
        # the fused kernels return the output in the memory layout of q ([B, S, H, D] storage seen as [B, H, S, D]):
        # the `transpose(1, 2).contiguous()` that follows in the models is then free
        if q.shape[-1] == v.shape[-1]:
            out = torch.empty_like(q)
        else:
            out = torch.empty(*q.shape[:-1], v.shape[-1], dtype=q.dtype, device=q.device)
        lse = torch.empty(q.shape[:-1], dtype=torch.float32, device=q.device)
        ctx.save_for_backward(q, k, v, out, lse)
        if _ACTIVE_COST[0] is not None:
            _ACTIVE_COST[0].on_dense_attention(q, k, backward=False)
        return out

    @staticmethod
    def backward(ctx, g):
        q, k, v, _, _ = ctx.saved_tensors
        if _ACTIVE_COST[0] is not None:
            _ACTIVE_COST[0].on_dense_attention(q, k, backward=True)
        return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _sdpa_stand_in(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False):
    return _FlashStandIn.apply(q, k, v)


def _example_inputs_on_meta(trainer_config, model_config):
    """For loaders that feed more than tokens (images): one batch from the recipe's own SYNTHETIC loader, shapes only.
    → (input dict on the meta device, labels on the meta device) or None when tokens alone are the input."""
    dl = trainer_config.dataloader
    if getattr(dl, "dataset", None) != "synthetic" or not type(dl).__name__.startswith("MultiModal"):
        return None
    from titan_b200.data.synthetic import build_dataloader

    loader = build_dataloader(dl, model_config=model_config, training=trainer_config.training, dp_rank=0,
                              dp_world_size=1)
    batch, labels = next(iter(loader))
    to_meta = lambda t: torch.empty_like(t, device="meta") if isinstance(t, torch.Tensor) else t   # noqa: E731
    return {k: to_meta(v) for k, v in batch.items()}, to_meta(labels)


def _measure_timeline(model, model_config, training, loss_fn, num_mtp: int, grad_keep: dict,
                      cost=None, example=None) -> tuple[int, int]:
    """One forward + backward on meta tensors.  Returns (peak bytes of activations + gradients-so-far, gradient
    bytes inside that peak).  ``grad_keep[param] = fraction`` of a parameter's gradient that stays on this rank once
    it has been reduced (1 on one GPU, 1 / fsdp under FSDP, ...)."""
    import torch.nn.functional as F

    b, s = training.local_batch_size, training.seq_len
    tokens = torch.empty(b, s + num_mtp, dtype=torch.int64, device="meta")   # MTP depths read the look-ahead tokens
    labels = torch.empty(b, s + num_mtp, dtype=torch.int64, device="meta")
    real_sdpa = F.scaled_dot_product_attention
    F.scaled_dot_product_attention = _sdpa_stand_in
    hooks = []
    grads_live = {"bytes": 0, "at_peak": 0, "peak": 0}
    from titan_b200.ops import _lib

    try:
        # the wrappers take their kernel code paths on the meta tensors (same buffers and saved tensors as on a GPU)
        # with every launch a no-op
        _ACTIVE_COST[0] = cost
        with _lib.no_launch(on_call=cost.on_library_call if cost is not None else None), \
                MetaMemoryTracker(cost) as tr:
            def on_grad(p):
                keep = grad_keep.get(p, 1.0)
                n = p.grad.numel() * p.grad.element_size()
                tr.reweight(p.grad, keep)
                grads_live["bytes"] += int(n * keep)
                if tr.peak > grads_live["peak"]:
                    # the gradient was created at full size before this hook ran: the new peak holds all of it
                    grads_live["peak"], grads_live["at_peak"] = tr.peak, grads_live["bytes"] - int(n * keep) + n

            for p in model.parameters():
                if p.requires_grad:
                    hooks.append(p.register_post_accumulate_grad_hook(on_grad))
            if example is not None:
                batch, labels = example
                batch = dict(batch)
                out = model(batch.pop("input"), **batch)
            else:
                out = model(tokens)
            loss = loss_fn(out, labels)
            del out
            loss.backward()
            peak = tr.peak
    finally:
        _ACTIVE_COST[0] = None
        F.scaled_dot_product_attention = real_sdpa
        for h in hooks:
            h.remove()
    at_peak = grads_live["at_peak"] if grads_live["peak"] == peak else 0
    for p in model.parameters():
        p.grad = None
    return peak, at_peak


def estimate(trainer_config, world_size: int, *, link_gbs: float = 770.0) -> MemoryReport:
    from titan_b200.parallel.parallel_dims import ParallelDims
    from titan_b200.protocols.converter import ModelConvertersContainer
    from titan_b200.protocols.model_spec import get_model_spec

    cfg = trainer_config
    par = cfg.parallelism
    pd = ParallelDims(
        dp_replicate=par.data_parallel_replicate_degree, dp_shard=par.data_parallel_shard_degree,
        cp=par.context_parallel_degree, tp=par.tensor_parallel_degree, pp=par.pipeline_parallel_degree,
        ep=par.expert_parallel_degree, etp=par.expert_tensor_parallel_degree, world_size=world_size)
    spec = get_model_spec(cfg.model.name, cfg.model.flavor)
    mc = spec.model
    for key, value in cfg.model.overrides.items():
        setattr(mc, key, value)
    mc.update_from_config(trainer_config=cfg)
    store_dt = _DT[cfg.training.dtype]
    old = torch.get_default_dtype()
    torch.set_default_dtype(store_dt)
    try:
        with torch.device("meta"):
            model = mc.build()
    finally:
        torch.set_default_dtype(old)
    ModelConvertersContainer(cfg.model_converters.converters, model_spec=spec, trainer_config=cfg).convert(model)
    notes = []

    # ---- static shards
    fsdp = pd.dp_shard * pd.cp
    total = local = 0.0
    largest_unit = 0.0
    per_layer: dict[str, float] = {}
    expert_local = 0.0
    for name, p in model.named_parameters():
        n = p.numel()
        total += n
        if _is_expert(name):
            shard = pd.efsdp * pd.ep * (pd.etp if pd.etp_enabled else 1)
            expert_local += n / shard / pd.pp
        else:
            tp_sharded = p.dim() >= 2 and pd.tp_enabled
            shard = fsdp * (pd.tp if tp_sharded else 1)
        local += n / shard / pd.pp
        unit = name.split(".")[1] if name.startswith("layers.") else name.split(".")[0]
        gathered = n / ((pd.ep * (pd.etp if pd.etp_enabled else 1)) if _is_expert(name)
                        else (pd.tp if (p.dim() >= 2 and pd.tp_enabled) else 1))
        per_layer[unit] = per_layer.get(unit, 0.0) + gathered
    largest_unit = max(per_layer.values()) if per_layer else 0.0
    sb = torch.empty((), dtype=store_dt).element_size()
    param_dt = _DT[cfg.training.mixed_precision_param]
    pb = torch.empty((), dtype=param_dt).element_size()
    rb = torch.empty((), dtype=_DT[cfg.training.mixed_precision_reduce]).element_size()
    bytes_params = int(local * sb)
    bytes_grads = int(local * sb)
    # two moments: fp32 for the framework's fused AdamW, the parameters' storage dtype for the library implementations
    # (`torch.optim.AdamW` allocates its state with `zeros_like(param)`)
    moment_bytes = 4 if cfg.optimizer.implementation == "b200_fused" else sb
    opt_bytes = int(local * 2 * moment_bytes)
    if cfg.optimizer.name == "Muon":
        opt_bytes = int(local * 4)
        notes.append("Muon keeps one momentum buffer for matrix params (AdamW moments for the rest are a few %)")
    on_host = cfg.optimizer.swap_optimizer or cfg.optimizer.virtual_optimizer
    bytes_opt_dev = 0 if on_host else opt_bytes
    bytes_opt_host = opt_bytes if on_host else 0
    if cfg.optimizer.swap_optimizer:
        # one slice of the state is resident at a time while the step streams through
        bytes_opt_dev = int(opt_bytes / max(cfg.optimizer.swap_optimizer_times, 1)) * 2
    peer_rs = fsdp > 1 and getattr(par, "fsdp_reduce_scatter", "nccl") != "nccl" and fsdp <= 8
    wire = pb if peer_rs else rb               # bytes per element of the gradient bucket
    bytes_fsdp = bytes_gathered = 0
    if fsdp > 1:
        # next unit's all-gather output + one unit's unsharded gradients + its reduction bucket and output
        bytes_fsdp = int(largest_unit * pb + largest_unit * pb + largest_unit * wire + largest_unit * rb / fsdp)
        dense_gathered = sum(v for k, v in per_layer.items())
        if par.fsdp_reshard_after_forward == "never":
            bytes_gathered = int(dense_gathered * pb)
        else:
            bytes_gathered = int(min(dense_gathered, 2 * largest_unit) * pb)
        if sb != pb:
            notes.append("parameters are stored in a wider dtype than they are gathered in")

    # ---- forward + backward timeline on meta tensors
    loss_fn = spec.build_loss_fn(None, trainer_config=cfg) if spec.build_loss_fn else None
    if cfg.activation_checkpoint.mode != "none":
        from titan_b200.parallel.activation_checkpoint import apply_ac

        apply_ac(model, cfg.activation_checkpoint)
    grad_keep = {}
    for name, p in model.named_parameters():
        if _is_expert(name):
            shard = pd.efsdp * pd.ep * (pd.etp if pd.etp_enabled else 1)
        else:
            shard = fsdp * (pd.tp if (p.dim() >= 2 and pd.tp_enabled) else 1)
        grad_keep[p] = 1.0 / shard
    if fsdp > 1 and store_dt != param_dt:
        model.to(param_dt)   # FSDP computes on gathered copies in the parameter dtype: so do the activations
    grads_at_peak = 0
    # Fused expert parallelism sizes every expert-major buffer of a layer for the rows an owner rank may receive
    # (capacity factor x the balanced load), not for the balanced load itself, and keeps two receive buffers of that
    # size in symmetric memory.  The meta model routes locally, so its row capacity is replaced for the run.
    from titan_b200.ops import moe as moe_ops

    real_capacity = moe_ops.capacity_for
    bytes_ep_workspace = 0
    fused_ep = pd.ep_enabled and par.expert_parallel_comm_backend == "fused_p2p"
    if fused_ep:
        from titan_b200.ops.moe_comm import capacity_per_owner

        factor = float(par.expert_parallel_capacity_factor)
        moe_ops.capacity_for = lambda pairs, experts: capacity_per_owner(pairs, max(experts // pd.ep, 1), pd.ep, factor)
        tok = cfg.training.local_batch_size * cfg.training.seq_len // max(pd.cp * pd.tp, 1)
        topk = getattr(getattr(mc, "moe_args", None), "top_k", getattr(mc, "top_k", 1))
        n_exp = getattr(getattr(mc, "moe_args", None), "num_experts", getattr(mc, "num_experts", pd.ep))
        bytes_ep_workspace = 2 * moe_ops.capacity_for(tok * topk, n_exp) * mc.dim * pb
        notes.append(f"fused expert parallelism: expert-major buffers hold {factor:g}x the balanced rows; "
                     f"{bytes_ep_workspace / GIB:.2f} GiB of symmetric receive buffers")
    from titan_b200.simulator.cost import StepCost

    cost = StepCost()
    if fused_ep:
        # the grouped products only touch the rows in use, not the capacity the buffers are sized for
        tok_pairs = cfg.training.local_batch_size * cfg.training.seq_len * max(int(topk), 1)
        cost.grouped_rows_scale = real_capacity(tok_pairs, n_exp) / max(moe_ops.capacity_for(tok_pairs, n_exp), 1)
    try:
        dyn, grads_at_peak = _measure_timeline(model, mc, cfg.training, loss_fn, cfg.training.num_mtp_modules,
                                               grad_keep, cost, _example_inputs_on_meta(cfg, mc))
        act = max(dyn - grads_at_peak, 0)
    except Exception as e:  # an op without a meta kernel: fall back to a closed-form bound
        L, d = mc.n_layers, mc.dim
        tok = cfg.training.local_batch_size * cfg.training.seq_len
        per_layer_act = {"full": 1, "selective": 10, "none": 24}[cfg.activation_checkpoint.mode]
        act = int(tok * d * pb * per_layer_act * L + tok * mc.vocab_size * (pb + 4))
        notes.append(f"activation term from the closed-form bound ({type(e).__name__}: {str(e)[:80]})")
        cost = None   # no traced step: no step-time estimate either
    finally:
        moe_ops.capacity_for = real_capacity
    act = int(act / (pd.tp * pd.cp) / pd.pp)
    grads_at_peak = int(grads_at_peak / pd.pp)
    dyn_peak = act + grads_at_peak
    if fsdp > 1 and par.fsdp_reshard_after_forward == "never":
        # nothing is gathered in backward, and the first reduction starts only after the last layer's backward has
        # freed that layer's activations: only what the reduction needs beyond them adds to the peak
        n_units = max(getattr(mc, "n_layers", 1), 1)
        bytes_fsdp = max(0, int(largest_unit * (pb + wire) + largest_unit * rb / fsdp) - act // n_units)

    # ---- link traffic per step (bytes sent+received by one rank)
    comm = {}
    if fsdp > 1:
        dense_total = (total - sum(p.numel() for n, p in model.named_parameters() if _is_expert(n))) / pd.pp
        gathers = 2 if par.fsdp_reshard_after_forward != "never" else 1
        comm["fsdp_all_gather"] = dense_total / (pd.tp if pd.tp_enabled else 1) * pb * gathers * (fsdp - 1) / fsdp
        comm["fsdp_reduce_scatter"] = dense_total / (pd.tp if pd.tp_enabled else 1) * rb * (fsdp - 1) / fsdp
    if pd.tp_enabled:
        tok = cfg.training.local_batch_size * cfg.training.seq_len / pd.cp
        per_layer_bytes = tok * mc.dim * pb * (pd.tp - 1) / pd.tp
        comm["tp_sp_collectives"] = per_layer_bytes * 4 * 2 * mc.n_layers / pd.pp  # 2 AG + 2 RS, fwd + bwd
    if pd.ep_enabled:
        tok = cfg.training.local_batch_size * cfg.training.seq_len / pd.cp
        topk = getattr(getattr(mc, "moe_args", None), "top_k", getattr(mc, "top_k", 1))
        n_moe = getattr(mc, "n_layers", 0) - getattr(mc, "n_dense_layers", 0)
        comm["ep_all_to_all"] = tok * topk * mc.dim * pb * (pd.ep - 1) / pd.ep * 4 * n_moe / pd.pp
    seconds = sum(comm.values()) / (link_gbs * 1e9)

    # the optimizer step runs after backward with every local gradient present and no activation left
    at_step = bytes_params + bytes_grads + bytes_opt_dev
    bytes_fsdp += bytes_ep_workspace
    # ---- step time: traced operators (sequence- / context- / pipeline-parallel ranks share them), optimizer, the
    #      part of the collectives that compute does not hide
    step_s = tok_s = 0.0
    by_kind: dict = {}
    flops_rank = 0.0
    n_ops = 0
    if cost is not None:
        share = pd.tp * pd.cp * pd.pp
        compute_s = cost.seconds / share
        by_kind = {k: v / share for k, v in cost.by_kind.items()}
        if pd.cp > 1 and "indexer scoring" in by_kind:
            # all-gather context parallelism: rank r scores its queries against (r + 1) / cp of the keys, and the
            # step waits for the last rank, which has (2 - 1 / cp) times the average number of pairs
            extra = by_kind["indexer scoring"] * (1.0 - 1.0 / pd.cp)
            by_kind["indexer scoring"] += extra
            compute_s += extra
        flops_rank = cost.flops / share
        n_ops = cost.launches + cost.free_ops
        cost.seconds, cost.by_kind = 0.0, {}
        cost.add_optimizer_step(local, sb, 4 if cfg.optimizer.implementation == "b200_fused" else sb)
        if cfg.optimizer.swap_optimizer:
            cost.add_optimizer_swap(bytes_opt_host)
        cost.exposed_collectives(comm, link_gbs)
        by_kind.update(cost.by_kind)
        device_s = compute_s + cost.seconds
        host_s = n_ops * cost.peaks.host_s_per_operator
        step_s = max(device_s, host_s)
        if host_s > device_s:
            by_kind = {"host (operator dispatch)": host_s, **by_kind}
            notes.append(f"the step is host-bound: {n_ops:,} operators at "
                         f"{cost.peaks.host_s_per_operator * 1e6:.0f} us each exceed {device_s * 1e3:.0f} ms of kernels")
        if cost.unpriced:
            notes.append(f"{cost.unpriced} operators could not be priced and count as free in the step time")
        if pd.ep_enabled:
            notes.append("step time excludes the waits between expert-parallel ranks at every dispatch / combine: "
                         "a lower bound for expert-parallel recipes")
        tokens = cfg.training.local_batch_size * cfg.training.seq_len * pd.dp_replicate * pd.dp_shard
        tok_s = tokens / step_s if step_s > 0 else 0.0
    total_bytes = max(bytes_params + bytes_opt_dev + bytes_fsdp + bytes_gathered + dyn_peak, at_step)
    budget = int(cfg.memory_sim.hbm_budget_gib * 1e9)
    return MemoryReport(
        world_size=world_size,
        parallelism={"dp_replicate": pd.dp_replicate, "dp_shard": pd.dp_shard, "cp": pd.cp, "tp": pd.tp, "pp": pd.pp,
                     "ep": pd.ep, "etp": pd.etp},
        params_total=int(total), params_local=int(local), bytes_params=bytes_params, bytes_grads=bytes_grads,
        bytes_optimizer_device=bytes_opt_dev, bytes_optimizer_host=bytes_opt_host, bytes_fsdp_buffers=bytes_fsdp,
        bytes_activations=act, bytes_total=total_bytes, budget_bytes=budget, fits=total_bytes <= budget,
        bytes_gathered_params=bytes_gathered, bytes_dynamic_peak=dyn_peak, bytes_grads_at_peak=grads_at_peak,
        comm_bytes_per_step={k: float(v) for k, v in comm.items()}, comm_seconds_per_step=seconds, notes=notes,
        step_seconds_estimate=step_s, tokens_per_second_estimate=tok_s, flops_per_rank_step=flops_rank,
        seconds_by_kind={k: round(v, 6) for k, v in sorted(by_kind.items(), key=lambda kv: -kv[1])},
        operators_per_step=n_ops)


def run_from_config(trainer_config) -> MemoryReport:
    import os

    world = int(os.environ.get("NGPU", os.environ.get("WORLD_SIZE", "1")))
    try:
        rep = estimate(trainer_config, world)
    except ValueError as e:
        if "world_size" in str(e) and "NGPU" not in os.environ and "WORLD_SIZE" not in os.environ:
            raise ValueError(f"{e}; the memory estimate takes the job size from NGPU (or WORLD_SIZE): "
                             f"e.g. NGPU=8 python -m titan_b200.entry ... --memory_sim.enable") from None
        raise
    path = trainer_config.memory_sim.report_path
    if path:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            f.write(rep.to_json())
    return rep
