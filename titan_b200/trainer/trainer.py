"""The training loop.

`Trainer(config)` builds, in order: process group → `ParallelDims` + meshes →
dataloader → model on the meta device → converters → `parallelize_fn` (or the
pipeline split) → materialise + init → loss → optimizer → LR schedule →
checkpoint manager.  `train()` then loops: garbage collection tick, gradient
accumulation over microbatches (`forward_backward_step`), gradient clipping,
optimizer + scheduler step, metrics, checkpoint, profiler step.

Loss normalisation: every microbatch loss is a *sum* over tokens divided by the
number of valid tokens of the whole global batch (all data-parallel ranks × all
accumulation steps) *before* backward, so pipeline and non-pipeline runs produce
identical gradients.

Parity: the trainer surface the reference patches (`__init__`, `init_distributed`,
`train`, `train_step`, `forward_backward_step(input_dict, labels, global_valid_tokens)`,
`post_dataloading_process → (inputs, labels, extra_inputs, extra_kwargs)`, `close`):
torchtitan_npu/train.py:22-175, patches/torchtitan/pp_loss_normalize.py:50-124,
patches/torchtitan/_trainer_config_stash.py:38-85, entry.py:113-132.
"""

from __future__ import annotations

import contextlib
import os
import time
from typing import Any

import torch
import torch.distributed as dist
import torch.nn as nn

from titan_b200.lowp.mx_linear import invalidate_weight_cache
from titan_b200.checkpoint.manager import CheckpointManager
from titan_b200.data.synthetic import build_dataloader
from titan_b200.optim.containers import build_lr_schedulers, build_optimizers
from titan_b200.parallel import utils as dist_utils
from titan_b200.parallel.parallel_dims import ParallelDims
from titan_b200.protocols.converter import ModelConvertersContainer
from titan_b200.protocols.model_spec import get_model_spec
from titan_b200.trainer import stash
from titan_b200.trainer.gc import GarbageCollection
from titan_b200.trainer.kernel_status import KernelStatusMonitor
from titan_b200.trainer.loss import IGNORE_INDEX
from titan_b200.trainer.metrics import MetricsProcessor
from titan_b200.trainer.profiling import maybe_enable_memory_snapshot, maybe_enable_profiling
from titan_b200.utils.logging import init_logger, logger

__all__ = ["Trainer", "TrainState", "get_grad_accumulation_steps"]


class TrainState:
    def __init__(self):
        self.step = 0
        self.ntokens_seen = 0

    def state_dict(self) -> dict[str, Any]:
        return {"step": torch.tensor(self.step, dtype=torch.int64),
                "ntokens_seen": torch.tensor(self.ntokens_seen, dtype=torch.int64)}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        self.step = int(sd["step"])
        self.ntokens_seen = int(sd.get("ntokens_seen", 0))


def get_grad_accumulation_steps(training, parallel_dims: ParallelDims) -> int:
    """Accumulation steps implied by global / local batch sizes (PP feeds whole local batches)."""
    dp = parallel_dims.dp_replicate * parallel_dims.dp_shard
    gbs = training.global_batch_size
    if gbs < 0:
        return 1
    denom = training.local_batch_size * dp
    if gbs % denom != 0:
        raise ValueError(f"global_batch_size {gbs} must be a multiple of local_batch_size * dp = {denom}")
    return gbs // denom


class Trainer:
    def __init__(self, config):
        init_logger()
        self.config = config
        stash.set_trainer_config(config)
        cfg = config
        if cfg.debug.print_config or cfg.job.print_config:
            logger.info("config: %s", cfg.to_dict())

        self.device = self._pick_device()
        world_size = self.init_distributed()
        par = cfg.parallelism
        self.parallel_dims = ParallelDims(
            dp_replicate=par.data_parallel_replicate_degree, dp_shard=par.data_parallel_shard_degree,
            cp=par.context_parallel_degree, tp=par.tensor_parallel_degree, pp=par.pipeline_parallel_degree,
            ep=par.expert_parallel_degree, etp=par.expert_tensor_parallel_degree, world_size=world_size,
            dedicated_ep_group=par.dedicated_ep_group,
        )
        pd = self.parallel_dims
        stash.set_active_parallel_dims(pd)
        if world_size > 1 or dist.is_initialized():
            pd.build_mesh(self.device.type)
        rank = dist.get_rank() if dist.is_initialized() else 0
        self.rank = rank
        coord = pd.coordinate(rank)
        self.dp_rank = coord["dp_replicate"] * pd.dp_shard + coord["dp_shard"]
        self.dp_degree = pd.dp_degree

        seed = cfg.debug.seed if cfg.debug.seed is not None else cfg.training.seed
        dist_utils.set_determinism(seed, cfg.debug.deterministic or cfg.training.deterministic, parallel_dims=pd,
                                   warn_only=cfg.debug.deterministic_warn_only)
        if torch.cuda.is_available():
            torch.backends.cuda.matmul.allow_tf32 = cfg.training.allow_tf32
            torch.backends.cudnn.allow_tf32 = cfg.training.allow_tf32
            if cfg.training.device_memory_ratio < 1.0:
                torch.cuda.set_per_process_memory_fraction(cfg.training.device_memory_ratio)
        self.gc_handler = GarbageCollection(gc_freq=cfg.training.gc_freq, debug=cfg.training.gc_debug)

        # ---- model spec, dataloader
        self.model_spec = get_model_spec(cfg.model.name, cfg.model.flavor)
        model_config = self.model_spec.model
        for key, value in cfg.model.overrides.items():
            if not hasattr(model_config, key):
                raise AttributeError(f"model config of {cfg.model.name}/{cfg.model.flavor} has no field {key!r}")
            setattr(model_config, key, value)
        model_config.update_from_config(trainer_config=cfg)
        self.model_config = model_config
        self.tokenizer = self._build_tokenizer()
        self.dataloader = build_dataloader(cfg.dataloader, model_config=model_config, training=cfg.training,
                                           dp_rank=self.dp_rank, dp_world_size=self.dp_degree,
                                           tokenizer=self.tokenizer)

        # ---- model on meta, converters
        store_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[cfg.training.dtype]
        with torch.device("meta"), _default_dtype(store_dtype):
            model = model_config.build()
        self.model_converters = ModelConvertersContainer(cfg.model_converters.converters, model_spec=self.model_spec,
                                                         trainer_config=cfg)
        self.model_converters.convert(model)
        if cfg.model_converters.print_after_conversion:
            logger.info("%s", model)
        nparams, flops_per_token = model_config.get_nparams_and_flops(model, cfg.training.seq_len)
        self.nparams, self.flops_per_token = nparams, flops_per_token
        logger.info("model %s %s: %s parameters", self.model_spec.name, self.model_spec.flavor, f"{nparams:,}")

        self.metrics_processor = MetricsProcessor(cfg.metrics, parallel_dims=pd, dump_folder=cfg.job.dump_folder,
                                                  quantized=self._is_quantized(), rank=rank)
        self.metrics_processor.num_flops_per_token = flops_per_token

        # ---- loss
        build_loss = self.model_spec.build_loss_fn
        self.loss_fn = build_loss(cfg.compile, trainer_config=cfg)

        # ---- batch bookkeeping
        self.gradient_accumulation_steps = get_grad_accumulation_steps(cfg.training, pd)
        if cfg.training.global_batch_size < 0:
            cfg.training.global_batch_size = cfg.training.local_batch_size * self.dp_degree

        # ---- parallelise + materialise
        init_device = "cpu" if cfg.training.enable_cpu_offload else self.device.type
        self.pp_schedule = None
        self.pp_has_first_stage = self.pp_has_last_stage = True
        if pd.pp_enabled:
            if self.model_spec.pipelining_fn is None:
                raise RuntimeError(f"pipeline parallelism is not supported for {self.model_spec.name}")
            (self.pp_schedule, self.model_parts, self.pp_has_first_stage,
             self.pp_has_last_stage) = self.model_spec.pipelining_fn(
                model, parallel_dims=pd, trainer_config=cfg, device=self.device, model_config=model_config,
                parallelize_fn=self.model_spec.parallelize_fn, loss_fn=self._pp_loss_fn(),
            )
            del model
            for m in self.model_parts:
                m.to_empty(device=init_device)
                with torch.no_grad():
                    m.init_states(buffer_device=self.device)
                m.train()
        else:
            model = self.model_spec.parallelize_fn(
                model, parallel_dims=pd, training=cfg.training, model_converters=cfg.model_converters,
                parallelism=par, compile_config=cfg.compile, ac_config=cfg.activation_checkpoint,
                dump_folder=cfg.job.dump_folder,
            )
            model.to_empty(device=init_device)
            with torch.no_grad():
                model.init_states(buffer_device=self.device)
            model.train()
            self.model_parts = [model]
        # losses are normalised by the global token count, so gradients must be SUMMED over
        # data-parallel ranks, not averaged
        _disable_fsdp_gradient_division(self.model_parts)

        # ---- optimizer, schedule, hooks
        self.optimizers = build_optimizers(self.model_parts, cfg.optimizer, pd, cuda_graph=cfg.compile.cuda_graphs)
        if self.model_spec.post_optimizer_build_fn is not None:
            self.model_spec.post_optimizer_build_fn(self.optimizers, self.model_parts, pd)
        self.lr_schedulers = build_lr_schedulers(self.optimizers, cfg.lr_scheduler, cfg.training.steps)
        self.optimizers.register_step_post_hook(
            lambda *a, **k: self.model_converters.post_optimizer_hook(self.model_parts))

        # ---- checkpoint
        self.train_state = TrainState()
        adapter = None
        if self.model_spec.state_dict_adapter is not None:
            adapter = self.model_spec.state_dict_adapter(model_config, cfg.model.hf_assets_path)
        self.checkpointer = CheckpointManager(
            dataloader=self.dataloader, model_parts=self.model_parts, optimizers=self.optimizers,
            lr_schedulers=self.lr_schedulers, states={"train_state": self.train_state}, config=cfg.checkpoint,
            sd_adapter=adapter, base_folder=cfg.job.dump_folder,
        )
        self.step = 0
        self.ntokens_seen = 0
        self.loss_history: list[float] = []
        self._cache_emptied = False
        self.kernel_status = KernelStatusMonitor()
        logger.info("trainer ready: world %d, dp_shard %d, dp_replicate %d, tp %d, cp %d, pp %d, ep %d; "
                    "global batch %d, grad-accum %d", world_size, pd.dp_shard, pd.dp_replicate, pd.tp, pd.cp, pd.pp,
                    pd.ep, cfg.training.global_batch_size, self.gradient_accumulation_steps)

    # ------------------------------------------------------------------ setup helpers
    def _pick_device(self) -> torch.device:
        if torch.cuda.is_available() and self.config.comm.mode != "fake_backend":
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            return torch.device("cuda", local)
        if torch.cuda.is_available():
            return torch.device("cuda", 0)
        return torch.device("cpu")

    def init_distributed(self) -> int:
        ws_env = int(os.environ.get("WORLD_SIZE", "1"))
        if self.config.comm.mode == "fake_backend" or ws_env > 1 or dist.is_initialized():
            return dist_utils.init_distributed(self.config.comm, world_size=ws_env,
                                               base_folder=self.config.job.dump_folder)
        return 1

    def _build_tokenizer(self):
        from titan_b200.config.configs import SyntheticDataLoaderConfig

        if isinstance(self.config.dataloader, SyntheticDataLoaderConfig):
            return None
        if getattr(self.config.dataloader, "dataset", None) == "synthetic":  # synthetic multimodal batches
            return None
        from titan_b200.data.tokenizer import build_tokenizer

        return build_tokenizer(self.config.model.tokenizer_path or self.config.model.hf_assets_path)

    def _is_quantized(self) -> bool:
        for c in self.config.model_converters.converters:
            name = getattr(c, "name", None) or type(c).__qualname__
            if any(t in str(name).lower() for t in ("mxfp8", "float8", "quantize")):
                return True
        return False

    def _pp_loss_fn(self):
        def fn(pred, labels):
            # divisor is refreshed every step before the schedule runs
            return self.loss_fn(pred, labels) / self._pp_loss_divisor

        self._pp_loss_divisor = 1.0
        return fn

    # ------------------------------------------------------------------ data
    def batch_generator(self, data_iterable):
        it = iter(data_iterable)
        while True:
            t0 = time.perf_counter()
            try:
                input_dict, labels = next(it)
            except StopIteration as e:
                raise RuntimeError("dataloader exhausted") from e
            self.metrics_processor.data_loading_times.append(time.perf_counter() - t0)
            ntok = labels.numel()
            self.ntokens_seen += ntok
            self.metrics_processor.ntokens_since_last_log += ntok
            dev = self.device
            input_dict = {k: (v.to(dev, non_blocking=True) if isinstance(v, torch.Tensor) else v)
                          for k, v in input_dict.items()}
            yield input_dict, labels.to(dev, non_blocking=True)

    def post_dataloading_process(self, input_dict: dict[str, torch.Tensor], labels: torch.Tensor):
        """→ (inputs, labels, extra_inputs, extra_kwargs); models/converters may override via hooks."""
        inputs = input_dict["input"]
        extra_inputs = {k: v for k, v in input_dict.items() if k != "input"}
        extra_kwargs: dict[str, Any] = {}
        for hook in stash.post_dataloading_hooks():
            inputs, labels, extra_inputs, extra_kwargs = hook(self, inputs, labels, extra_inputs, extra_kwargs)
        if getattr(self.model_config, "mask_type", None) == "varlen" and "positions" in extra_inputs:
            # document boundaries of the FULL sequence: built before any context-parallel slicing
            from titan_b200.models.common.varlen_attention import build_varlen_metadata

            extra_kwargs["attention_masks"] = build_varlen_metadata(extra_inputs["positions"])
        if getattr(self.model_config, "use_global_tnd", False) and "positions" in extra_inputs:
            # DeepSeek-V4 packed stream: every valid token of the batch in one [1, T] sequence
            if self.parallel_dims.pp_enabled or self.parallel_dims.cp_enabled:
                raise NotImplementedError("use_global_tnd excludes pipeline and context parallelism")
            from titan_b200.models.deepseek_v4.tnd import pack_global_tnd

            rows = tuple(inputs.shape)
            inputs, labels, packed = pack_global_tnd(inputs, labels, extra_inputs.pop("positions"), self.model_config)
            extra_kwargs.update(packed)
            if not getattr(self, "_tnd_logged", False):
                self._tnd_logged = True
                logger.info("global TND: batch %s packed into one stream of %d tokens, %d documents", rows,
                            inputs.shape[1], packed["attention_masks"].batch_size)
        if "positions" in extra_inputs:  # sliced together with the tokens under context parallelism
            extra_kwargs["positions"] = extra_inputs.pop("positions")
        if self.parallel_dims.cp_enabled:
            from titan_b200.parallel.context_parallel.sharding import prepare_context_parallel_input

            inputs, labels, extra_kwargs = prepare_context_parallel_input(
                inputs, labels, extra_kwargs, cp_mesh=self.parallel_dims.get_mesh("cp"), device=self.device,
                num_mtp_modules=self.config.training.num_mtp_modules,
                load_balancer=self.config.parallelism.context_parallel_load_balancer,
            )
        return inputs, labels, extra_inputs, extra_kwargs

    # ------------------------------------------------------------------ step
    def forward_backward_step(self, input_dict, labels, global_valid_tokens) -> torch.Tensor:
        inputs, labels, extra_inputs, extra_kwargs = self.post_dataloading_process(input_dict, labels)
        pd = self.parallel_dims
        if pd.pp_enabled:
            self._pp_loss_divisor = global_valid_tokens
            targets, losses = (labels, []) if self.pp_has_last_stage else (None, None)
            if self.pp_has_first_stage:
                self.pp_schedule.step(inputs, **extra_inputs, **extra_kwargs, target=targets, losses=losses)
            else:
                self.pp_schedule.step(**extra_kwargs, target=targets, losses=losses)
            if self.pp_has_last_stage:
                return torch.sum(torch.stack(losses)).detach().to(self.device)
            return torch.tensor(-1.0, device=self.device)
        model = self.model_parts[0]
        with self.train_context():
            pred = model(inputs, **extra_inputs, **extra_kwargs)
            loss = self.loss_fn(pred, labels) / global_valid_tokens
            del pred
            loss.backward()
        return loss.detach()

    def train_context(self):
        pd = self.parallel_dims
        if pd.tp_enabled and not self.config.parallelism.disable_loss_parallel:
            from torch.distributed.tensor.parallel import loss_parallel

            return loss_parallel()
        return contextlib.nullcontext()

    def train_step(self, data_iterator) -> None:
        self.optimizers.zero_grad()
        pd = self.parallel_dims
        micro = [next(data_iterator) for _ in range(self.gradient_accumulation_steps)]
        local_valid = sum((lab != IGNORE_INDEX).sum() for _, lab in micro).float()
        loss_mesh = pd.get_optional_mesh("loss") if dist.is_initialized() else None
        if loss_mesh is not None:
            # only data-parallel ranks hold distinct tokens; cp ranks hold slices of the same ones
            batch_mesh = pd.get_optional_mesh("dp")
            global_valid = local_valid.clone()
            if batch_mesh is not None:
                dist.all_reduce(global_valid, group=batch_mesh.get_group())
        else:
            global_valid = local_valid
        losses = [self.forward_backward_step(inp, lab, global_valid) for inp, lab in micro]

        params = [p for m in self.model_parts for p in m.parameters()]
        if pd.tp_enabled:
            dist_utils.reduce_partial_grads(params)
        if self.config.debug.grad_norm_breakdown:
            named = [(n, p) for m in self.model_parts for n, p in m.named_parameters() if p.grad is not None]
            pp_mesh = pd.get_optional_mesh("pp") if dist.is_initialized() else None
            for label, pick in (("experts", True), ("other", False)):
                gs = [p.grad for n, p in named if (".experts." in n) == pick]
                if gs:
                    logger.info("step %d grad norm of %s: %.4f", self.step, label,
                                float(dist_utils.get_total_norm_local(gs, 2.0, pp_mesh=pp_mesh)))
        opts = list(self.optimizers)
        fused_clip = opts if opts and all(hasattr(o, "grad_scale") for o in opts) else None
        grad_norm = dist_utils.clip_grad_norm_(
            params, self.config.training.max_norm, foreach=True,
            pp_mesh=pd.get_optional_mesh("pp") if dist.is_initialized() else None, ep_enabled=pd.ep_enabled,
            defer_scale_to=fused_clip,  # optimizers that apply the clip coefficient inside their update kernel
        )
        self.optimizers.step()
        # the fused optimizer kernels write weights through raw pointers (no version bump): quantised copies kept by
        # the low-precision expert path are stale from here on
        invalidate_weight_cache()
        self.lr_schedulers.step()
        loss = torch.sum(torch.stack(losses))
        self._last_loss = loss
        self._last_grad_norm = grad_norm

        mp = self.metrics_processor
        mp.steps_since_last_log += 1
        if not mp.should_log(self.step):
            self.kernel_status.poll(f"step {self.step}")
            return
        self.kernel_status.check(f"step {self.step}")  # the log below syncs anyway
        if loss_mesh is not None:
            if pd.pp_enabled and not self.pp_has_last_stage:
                loss = torch.zeros_like(loss)
            # `loss` is local_sum / global_valid_tokens, so SUM over (dp × cp) ranks is the global mean
            avg = dist_utils.dist_sum(loss, loss_mesh)
            mx = dist_utils.dist_max(loss * (global_valid / torch.clamp(local_valid, min=1)), loss_mesh)
        else:
            avg = mx = float(loss)
        gn = float(grad_norm.full_tensor() if hasattr(grad_norm, "full_tensor") else grad_norm)
        extra = {}
        for hook in stash.metrics_hooks():
            extra.update(hook(self) or {})
        self.loss_history.append(avg)
        mp.log(self.step, avg, mx, gn, extra_metrics=extra, loss_mesh=loss_mesh)

    # ------------------------------------------------------------------ loop
    def train(self) -> None:
        cfg = self.config
        self.checkpointer.load(step=cfg.checkpoint.load_step)
        self.step = self.train_state.step
        self.ntokens_seen = self.train_state.ntokens_seen
        if cfg.checkpoint.create_seed_checkpoint:
            if int(os.environ.get("WORLD_SIZE", "1")) != 1:
                raise RuntimeError("a seed checkpoint must be created by a single process")
            self.checkpointer.enable = True
            self.checkpointer.dcp_save(self.checkpointer._flattened_state(), self.checkpointer._step_dir(0),
                                       self.checkpointer.async_mode.DISABLED)
            logger.info("created seed checkpoint")
            return
        data_iterator = self.batch_generator(self.dataloader)
        logger.info("training starts at step %d", self.step + 1)
        with maybe_enable_profiling(cfg.profiling, global_step=self.step, base_folder=cfg.job.dump_folder,
                                    rank=self.rank) as prof, \
                maybe_enable_memory_snapshot(cfg.profiling, global_step=self.step,
                                             base_folder=cfg.job.dump_folder, rank=self.rank) as snap:
            self.metrics_processor.timer.start()
            while self.step < cfg.training.steps:
                self.step += 1
                self.gc_handler.run(self.step)
                if self.step == 1 and not self._cache_emptied and torch.cuda.is_available():
                    # staging buffers of a checkpoint load are dead weight from here on
                    torch.cuda.empty_cache()
                    self._cache_emptied = True
                self.train_step(data_iterator)
                self.train_state.step = self.step
                self.train_state.ntokens_seen = self.ntokens_seen
                if self.checkpointer._should_save(self.step, last_step=(self.step == cfg.training.steps)):
                    self.kernel_status.check(f"before the checkpoint of step {self.step}")
                self.checkpointer.save(self.step, last_step=(self.step == cfg.training.steps))
                if prof is not None:
                    prof.step()
                if snap is not None:
                    snap.step()
        logger.info("training completed")

    def close(self) -> None:
        if getattr(self, "checkpointer", None) is not None:
            self.checkpointer.close()
        if getattr(self, "metrics_processor", None) is not None:
            self.metrics_processor.close()
        stash.clear()


def _disable_fsdp_gradient_division(model_parts) -> None:
    from torch.distributed.fsdp import FSDPModule

    for part in model_parts:
        for m in part.modules():
            if isinstance(m, FSDPModule):
                m.set_gradient_divide_factor(1.0)
                # plain SUM reduce-scatter (no PREMUL_SUM op: gloo lacks it, and a factor of 1 needs none)
                m.set_force_sum_reduction_for_comms(True)


@contextlib.contextmanager
def _default_dtype(dtype: torch.dtype):
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        yield
    finally:
        torch.set_default_dtype(old)
