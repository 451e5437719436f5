"""Dataclass configuration tree of the trainer.

One tree (`TrainerConfig`) holds every knob.  Recipes are plain Python
functions that return a fully built `TrainerConfig` and compose with
`dataclasses.replace`; the CLI exposes every field as ``--section.field``.

Parity: the field set covers the reference's extensions
(torchtitan_npu/config/configs.py:57-309: swap / virtual / Muon optimizer
fields, `context_parallel_load_balancer`, MTP fields, step-range profiling,
checkpoint writer knobs, chat loader fields) plus the upstream trainer fields
its recipes set (torchtitan_npu/config/configs.py:311-378).
"""

from __future__ import annotations

import copy
from collections.abc import Callable
from dataclasses import dataclass, field, fields, is_dataclass, replace
from typing import Any, Literal

__all__ = [
    "JobConfig",
    "ProfilingConfig",
    "MetricsConfig",
    "ModelConvertersConfig",
    "OptimizerConfig",
    "LRSchedulerConfig",
    "TrainingConfig",
    "ParallelismConfig",
    "CheckpointConfig",
    "ActivationCheckpointConfig",
    "CompileConfig",
    "CommConfig",
    "DebugConfig",
    "MemorySimConfig",
    "TextDataLoaderConfig",
    "ChatEncoderConfig",
    "DSV4EncoderConfig",
    "ChatDataLoaderConfig",
    "SyntheticDataLoaderConfig",
    "MultiModalDataLoaderConfig",
    "TrainerConfig",
    "trainer_base_config",
    "debug_single_node_eq_pruned_config",
    "cpt_default_config",
    "sft_default_config",
    "deep_replace",
]


@dataclass(kw_only=True, slots=True)
class JobConfig:
    dump_folder: str = "./outputs"
    """Root folder for checkpoints, traces, snapshots and logs."""
    description: str = "titan_b200 training job"
    print_config: bool = False


@dataclass(kw_only=True, slots=True)
class ProfilingConfig:
    enable_profiling: bool = False
    save_traces_folder: str = "profile_traces"
    profile_freq: int = 10
    """Frequency mode: capture one window every `profile_freq` steps."""
    profiler_active: int = 1
    profiler_warmup: int = 3
    enable_memory_snapshot: bool = False
    save_memory_snapshot_folder: str = "memory_snapshot"
    # step-range mode (reference: config/configs.py:177-207)
    profile_step_start: int = 0
    """First profiled step; 0 keeps the frequency mode."""
    profile_step_end: int = 0
    """Last profiled step (exclusive); 0 means start + profiler_active."""
    profile_ranks: list[int] = field(default_factory=lambda: [-1])
    """Ranks to profile; [-1] profiles all ranks."""
    profile_record_shapes: bool = True
    profile_with_memory: bool = False
    profile_with_stack: bool = False
    enable_online_parse: bool = True
    """False leaves raw traces for offline parsing (no on_trace_ready handler)."""
    nvtx_ranges: bool = False
    """Emit NVTX ranges around fused kernels and trainer phases."""


@dataclass(kw_only=True, slots=True)
class MetricsConfig:
    log_freq: int = 10
    enable_tensorboard: bool = False
    save_tb_folder: str = "tb"
    save_for_all_ranks: bool = False
    disable_color_printing: bool = True
    device_timed: bool = True
    """Time steps with CUDA events (max over ranks) instead of host wall clock."""


@dataclass(kw_only=True, slots=True)
class ModelConvertersConfig:
    converters: list[Any] = field(default_factory=list)
    """Converter names or Config instances, applied in order after model build."""
    print_after_conversion: bool = False


@dataclass(kw_only=True, slots=True)
class OptimizerConfig:
    name: str = "AdamW"
    lr: float = 8e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    implementation: Literal["for-loop", "foreach", "fused", "b200_fused"] = "fused"
    """`b200_fused` selects the multi-tensor sm_100a AdamW kernel."""
    early_step_in_backward: bool = False
    # swap / virtual (reference: config/configs.py:57-129)
    swap_optimizer: bool = False
    """Keep optimizer state in pinned host memory; stream it through the GPU in slices during step()."""
    swap_optimizer_times: int = 16
    """Number of slices of the pipelined swap step."""
    virtual_optimizer: bool = False
    """Keep moments in host-mapped (device-addressable) memory up to a budget."""
    virtual_optimizer_size: float | list[float] | str | None = None
    """'all', GB per PP stage, or a per-stage list."""
    # Muon
    muon_lr: float | None = None
    muon_momentum: float = 0.95
    muon_enable_nesterov: bool = True
    muon_ns_steps: int = 5
    muon_adjust_lr_fn: Literal["original", "match_rms_adamw"] | None = "match_rms_adamw"
    muon_hybrid_ns: bool = False
    muon_extra_reduce_for_hsdp: bool = False
    """Average the Muon update over the `dp_replicate` ranks after Newton-Schulz (keeps HSDP replicas bit-identical)."""
    extra_param_group_split_rules: list[dict] | None = None
    swap_merge_buckets: int = 1


@dataclass(kw_only=True, slots=True)
class LRSchedulerConfig:
    warmup_steps: int = 200
    decay_ratio: float | None = None
    decay_type: Literal["linear", "sqrt", "cosine"] = "linear"
    min_lr_factor: float = 0.0


@dataclass(kw_only=True, slots=True)
class TrainingConfig:
    local_batch_size: int = 8
    global_batch_size: int = -1
    seq_len: int = 2048
    max_norm: float = 1.0
    steps: int = 10000
    enable_cpu_offload: bool = False
    mixed_precision_param: Literal["bfloat16", "float32"] = "bfloat16"
    mixed_precision_reduce: Literal["float32", "bfloat16"] = "float32"
    dtype: Literal["float32", "bfloat16"] = "float32"
    """Dtype the parameters are stored in (bf16 storage = "bf16 params")."""
    gc_freq: int = 50
    gc_debug: bool = False
    seed: int | None = None
    deterministic: bool = False
    # reference extensions (config/configs.py:149-175)
    device_memory_ratio: float = 1.0
    """Cap on the fraction of HBM the caching allocator may use."""
    num_mtp_modules: int = 0
    mtp_loss_weight: float = 0.3
    allow_tf32: bool = True
    """TF32 for fp32 matmul/conv (the CUDA analogue of the reference's HF32 flag)."""


@dataclass(kw_only=True, slots=True)
class ParallelismConfig:
    data_parallel_replicate_degree: int = 1
    data_parallel_shard_degree: int = -1
    fsdp_reshard_after_forward: Literal["default", "always", "never"] = "default"
    tensor_parallel_degree: int = 1
    disable_loss_parallel: bool = False
    enable_async_tensor_parallel: bool = False
    """Use the fused all-gather→GEMM / GEMM→reduce-scatter kernels for SP."""
    pipeline_parallel_degree: int = 1
    pipeline_parallel_schedule: str = "1F1B"
    pipeline_parallel_microbatch_size: int = 1
    pipeline_parallel_layers_per_stage: int | None = None
    pipeline_parallel_first_stage_less_layers: int = 1
    pipeline_parallel_last_stage_less_layers: int = 1
    context_parallel_degree: int = 1
    context_parallel_load_balancer: str | None = None
    """None = contiguous shards (required by Ulysses / DSA / compressor CP)."""
    context_parallel_rotate_method: str = "allgather"
    context_parallel_fused_projections: bool = False
    """Ulysses only: fold the head <-> sequence exchanges into the q/k/v and output projections (peer-memory GEMMs)."""
    expert_parallel_degree: int = 1
    expert_tensor_parallel_degree: int = 1
    expert_parallel_comm_backend: Literal["standard", "fused_p2p", "deepep", "hybridep", "torchao"] = "standard"
    """`fused_p2p` = in-kernel peer-memory dispatch/combine; `standard` = NCCL all-to-all."""
    expert_parallel_capacity_factor: float = 4.0
    """`fused_p2p` only: rows an owner rank's receive buffer holds, in multiples of the balanced load; the number of
    EP ranks makes it dropless.  A routing beyond it stops the step with a kernel status (nothing is dropped)."""
    fsdp_fused_collectives: bool = False
    """Fuse FSDP all-gather into the consuming GEMM and cast/scale into reduce-scatter."""
    fsdp_all_gather: Literal["auto", "nccl", "peer_memory"] = "auto"
    """Parameter all-gather of FSDP2: `nccl` = stock, `peer_memory` = copy-engine pulls from the peers' symmetric
    buffers (no SMs taken from the overlapping GEMMs), `auto` = `peer_memory` under the conditions of
    `fsdp_reduce_scatter`."""
    fsdp_reduce_scatter: Literal["auto", "nccl", "peer_memory", "nvls"] = "auto"
    """Gradient reduce-scatter of FSDP2: `nccl` = stock (fp32 bucket through NCCL), `peer_memory` = bf16 bucket in
    symmetric memory reduced by one kernel over NVLink peer loads, `nvls` = the same bucket summed inside the NVSwitch
    (`multimem.ld_reduce` through the slot's multicast address; falls back to peer loads where the fabric has no
    multicast), `auto` = `peer_memory` for CUDA jobs whose FSDP group is 2..8 GPUs of one node."""
    dedicated_ep_group: bool = True
    """Give EP its own communicator so FSDP and EP traffic overlap (reference train.py:136-175)."""


@dataclass(kw_only=True, slots=True)
class CheckpointConfig:
    enable: bool = False
    folder: str = "checkpoint"
    interval: int = 500
    load_step: int = -1
    initial_load_path: str | None = None
    initial_load_model_only: bool = True
    initial_load_in_hf: bool = False
    initial_load_in_hf_quantized: bool = False
    last_save_model_only: bool = True
    last_save_in_hf: bool = False
    export_dtype: Literal["float16", "bfloat16", "float32"] = "float32"
    load_only: bool = False
    keep_latest_k: int = 10
    exclude_from_loading: list[str] = field(default_factory=list)
    async_mode: Literal["disabled", "async", "async_with_pinned_mem"] = "disabled"
    create_seed_checkpoint: bool = False
    enable_first_step_checkpoint: bool = False
    enable_ft_dataloader_checkpoints: bool = True
    # writer knobs (reference: config/configs.py:210-230)
    sync_files: bool = True
    drop_page_cache_after_save: bool = False
    empty_cache_after_save: bool = True


@dataclass(kw_only=True, slots=True)
class ActivationCheckpointConfig:
    mode: Literal["none", "selective", "full"] = "selective"
    selective_ac_option: str = "op"
    """'op' = op-level policy, or an integer string N = checkpoint every Nth block."""
    selective_keep_swiglu: bool = False
    """Op-level policy: also keep the fused SwiGLU output (the down projection's input; hidden_dim * 2 bytes per token
    and layer).  Worth it for dense feed-forward blocks; MoE blocks would keep capacity-sized expert buffers."""
    per_op_sac_force_recompute_mm_shapes_by_fqns: list[str] = field(default_factory=lambda: ["moe.router.gate"])
    early_stop: bool = False
    preserve_rng_state: bool = False
    determinism_check: str = "default"


@dataclass(kw_only=True, slots=True)
class CompileConfig:
    enable: bool = False
    components: list[str] = field(default_factory=lambda: ["model", "loss"])
    backend: str = "inductor"
    cuda_graphs: bool = False
    """Record the fused AdamW step (every multi-tensor launch of every parameter group) as one CUDA graph and replay
    it each step; learning rate and bias corrections travel through a small device buffer.  Needs
    `optimizer.implementation = b200_fused`."""


@dataclass(kw_only=True, slots=True)
class CommConfig:
    mode: Literal["default", "fake_backend", "local_tensor"] = "default"
    """`fake_backend` runs one process that pretends to be NGPU ranks (dry run / simulator)."""
    backend: str | None = None
    """Override the process-group backend (nccl on CUDA, gloo on CPU by default)."""
    init_timeout_seconds: int = 300
    train_timeout_seconds: int = 100
    trace_buf_size: int = 20000
    """NCCL flight-recorder ring size; 0 disables it."""
    save_traces_folder: str = "comm_traces"
    save_traces_file_prefix: str = "rank_"


@dataclass(kw_only=True, slots=True)
class DebugConfig:
    seed: int | None = None
    deterministic: bool = False
    deterministic_warn_only: bool = False
    print_config: bool = False
    moe_force_load_balance: bool = False
    grad_norm_breakdown: bool = False
    """Log the gradient norm of the routed-expert weights and of everything else separately at every logged step."""


@dataclass(kw_only=True, slots=True)
class MemorySimConfig:
    enable: bool = False
    hbm_budget_gib: float = 180.0
    """Per-rank HBM budget the estimate is checked against."""
    report_path: str | None = None


@dataclass(kw_only=True, slots=True)
class TextDataLoaderConfig:
    dataset: str = "c4_test"
    dataset_path: str | None = None
    infinite: bool = True
    num_workers: int = 0
    pin_memory: bool = True


@dataclass(kw_only=True, slots=True)
class SyntheticDataLoaderConfig:
    """Uniform-random token ids from a fixed seed (no dataset / network needed)."""

    seed: int = 0
    vocab_size: int | None = None
    """None = the model's vocab size."""
    pin_memory: bool = True
    infinite: bool = True
    documents_per_row: int = 0
    """> 0: every row holds about this many packed documents and the batch carries their `positions`."""
    global_stream: bool = False
    """Draw the global batch from one stream and give each data-parallel rank its rows (N ranks x batch b then see the
    rows of 1 rank x batch N*b)."""


@dataclass(kw_only=True, slots=True)
class MultiModalDataLoaderConfig:
    """Image + text batches.  ``dataset="synthetic"`` draws random patches and tokens from a fixed seed; any other name
    is looked up in the multimodal dataset registry (needs the `datasets` package and local files)."""

    dataset: str = "synthetic"
    dataset_path: str | None = None
    max_patches_per_image: int = 256
    max_images_per_batch: int = 64
    patch_size: int = 16
    n_channels: int = 3
    seed: int = 0
    pin_memory: bool = True
    infinite: bool = True


@dataclass(kw_only=True, slots=True)
class ChatEncoderConfig:
    name: str = "chatml"


@dataclass(kw_only=True, slots=True)
class DSV4EncoderConfig(ChatEncoderConfig):
    name: str = "dsv4"
    encoding_path: str = ""
    """Path of the external `encoding_dsv4.py` implementation."""
    mode: Literal["chat", "thinking"] = "chat"
    drop_thinking: bool = True
    """Drop thinking blocks of earlier assistant turns (kept anyway when the conversation defines tools)."""
    reasoning_effort: Literal["max", "high"] | None = None


@dataclass(kw_only=True, slots=True)
class ChatDataLoaderConfig:
    dataset_path: str = ""
    load_dataset_kwargs: dict[str, Any] = field(default_factory=lambda: {"split": "train"})
    sample_processor: Callable | None = field(default=None, repr=False)
    chat_processor: str | None = None
    """Import path ``pkg.module:function`` of the sample → messages processor."""
    dataset_split: str | None = None
    data_files: str = ""
    dataset_config_name: str = ""
    chat_encoder: DSV4EncoderConfig | ChatEncoderConfig | None = None
    infinite: bool = True
    pack_sequences: bool = True
    num_workers: int = 0
    pin_memory: bool = True


@dataclass(kw_only=True, slots=True)
class ModelConfigRef:
    """Which model to build: a module under ``titan_b200.models`` and a flavor."""

    name: str = "llama3"
    flavor: str = "debugmodel"
    hf_assets_path: str = "./assets/hf"
    tokenizer_path: str | None = None
    overrides: dict[str, Any] = field(default_factory=dict)
    """Fields of the flavor's model config to replace (e.g. ``{"mask_type": "varlen"}``)."""


@dataclass(kw_only=True, slots=True)
class TrainerConfig:
    job: JobConfig = field(default_factory=JobConfig)
    model: ModelConfigRef = field(default_factory=ModelConfigRef)
    profiling: ProfilingConfig = field(default_factory=ProfilingConfig)
    metrics: MetricsConfig = field(default_factory=MetricsConfig)
    model_converters: ModelConvertersConfig = field(default_factory=ModelConvertersConfig)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    lr_scheduler: LRSchedulerConfig = field(default_factory=LRSchedulerConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    parallelism: ParallelismConfig = field(default_factory=ParallelismConfig)
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    activation_checkpoint: ActivationCheckpointConfig = field(default_factory=ActivationCheckpointConfig)
    compile: CompileConfig = field(default_factory=CompileConfig)
    comm: CommConfig = field(default_factory=CommConfig)
    debug: DebugConfig = field(default_factory=DebugConfig)
    memory_sim: MemorySimConfig = field(default_factory=MemorySimConfig)
    dataloader: TextDataLoaderConfig | ChatDataLoaderConfig | SyntheticDataLoaderConfig | MultiModalDataLoaderConfig = field(
        default_factory=SyntheticDataLoaderConfig
    )

    def build(self):
        """Construct the `Trainer` for this config."""
        from titan_b200.trainer.trainer import Trainer

        return Trainer(self)

    def to_dict(self) -> dict:
        return _to_dict(self)


def _to_dict(obj):
    if is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: _to_dict(getattr(obj, f.name)) for f in fields(obj)}
    if isinstance(obj, (list, tuple)):
        return [_to_dict(v) for v in obj]
    if isinstance(obj, dict):
        return {k: _to_dict(v) for k, v in obj.items()}
    if callable(obj) and not isinstance(obj, type):
        return getattr(obj, "__qualname__", repr(obj))
    return obj


def deep_replace(cfg, **changes):
    """`dataclasses.replace` on a deep copy.

    `replace` alone is shallow: nested lists/dicts stay shared between the
    base recipe and the derived one, so mutating one silently changes the other.
    """
    return replace(copy.deepcopy(cfg), **changes)


# --------------------------------------------------------------------------- base recipes
def trainer_base_config() -> TrainerConfig:
    """Production defaults shared by the DeepSeek recipes (reference config/configs.py:311-337)."""
    return TrainerConfig(
        debug=DebugConfig(print_config=True),
        metrics=MetricsConfig(log_freq=1),
        optimizer=OptimizerConfig(lr=1e-5, eps=1e-6, swap_optimizer=True),
        lr_scheduler=LRSchedulerConfig(warmup_steps=200, decay_ratio=0.8, decay_type="cosine", min_lr_factor=0.01),
        dataloader=TextDataLoaderConfig(),
        training=TrainingConfig(local_batch_size=1, global_batch_size=-1, seq_len=4096, steps=10000),
        parallelism=ParallelismConfig(fsdp_reshard_after_forward="always"),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
    )


def debug_single_node_eq_pruned_config(base: TrainerConfig) -> TrainerConfig:
    """Single-node debug preset on a pruned model (reference config/configs.py:340-352)."""
    return replace(
        base,
        debug=replace(base.debug, print_config=True, moe_force_load_balance=True),
        lr_scheduler=replace(base.lr_scheduler, warmup_steps=4),
        training=replace(base.training, global_batch_size=-1, steps=20),
        checkpoint=replace(base.checkpoint, load_step=0, load_only=True),
        compile=replace(base.compile, enable=False),
    )


def cpt_default_config(base: TrainerConfig) -> TrainerConfig:
    """Continued-pretraining preset: load HF weights once, long run (reference config/configs.py:355-369)."""
    return replace(
        base,
        comm=CommConfig(trace_buf_size=0),
        lr_scheduler=replace(base.lr_scheduler, warmup_steps=400),
        training=replace(base.training, steps=2000),
        checkpoint=replace(
            base.checkpoint, enable=True, load_step=0, interval=10000, load_only=True, initial_load_in_hf=True
        ),
    )


def sft_default_config(base: TrainerConfig) -> TrainerConfig:
    """SFT preset (reference config/configs.py:372-378)."""
    return replace(
        base,
        lr_scheduler=replace(base.lr_scheduler, warmup_steps=20),
        training=replace(base.training, global_batch_size=-1, steps=100),
        checkpoint=replace(base.checkpoint, interval=500, load_only=False, export_dtype="bfloat16"),
    )
