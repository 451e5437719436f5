"""Llama-3 recipes (``--module llama3 --config <name>``)."""

from titan_b200.config.configs import (
    ActivationCheckpointConfig,
    CheckpointConfig,
    LRSchedulerConfig,
    MetricsConfig,
    ModelConfigRef,
    ModelConvertersConfig,
    OptimizerConfig,
    ParallelismConfig,
    SyntheticDataLoaderConfig,
    TrainerConfig,
    TrainingConfig,
)
from titan_b200.protocols.converter import get_model_converter_config

_FUSED = ["b200_rms_norm", "b200_rope", "b200_swiglu", "b200_cross_entropy"]


def _fused_converters():
    return [get_model_converter_config(n) for n in _FUSED]


def llama3_debugmodel() -> TrainerConfig:
    """dim 256 / 6 layers; runs on CPU (gloo) or one GPU in seconds."""
    return TrainerConfig(
        model=ModelConfigRef(name="llama3", flavor="debugmodel"),
        metrics=MetricsConfig(log_freq=1),
        optimizer=OptimizerConfig(name="AdamW", lr=8e-4, implementation="for-loop"),
        lr_scheduler=LRSchedulerConfig(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0),
        training=TrainingConfig(local_batch_size=4, seq_len=512, steps=10, mixed_precision_param="float32",
                                mixed_precision_reduce="float32", dtype="float32"),
        dataloader=SyntheticDataLoaderConfig(seed=0),
        parallelism=ParallelismConfig(data_parallel_shard_degree=-1),
        checkpoint=CheckpointConfig(enable=False, interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="2"),
    )


def llama3_debugmodel_b200() -> TrainerConfig:
    """Debug model with every fused sm_100a op switched on (needs a B200)."""
    cfg = llama3_debugmodel()
    cfg.model_converters = ModelConvertersConfig(converters=_fused_converters())
    cfg.optimizer.implementation = "b200_fused"
    cfg.training.mixed_precision_param = "bfloat16"
    cfg.training.dtype = "bfloat16"
    return cfg


def llama3_8b() -> TrainerConfig:
    """Llama-3 8B pretraining: FSDP2, bf16 params/compute, fp32 reduce, seq 8192, local batch 1, selective
    activation checkpointing (contractions and attention kept, element-wise work recomputed), AdamW."""
    return TrainerConfig(
        model=ModelConfigRef(name="llama3", flavor="8B"),
        metrics=MetricsConfig(log_freq=10),
        optimizer=OptimizerConfig(name="AdamW", lr=3e-4, eps=1e-8, implementation="b200_fused"),
        lr_scheduler=LRSchedulerConfig(warmup_steps=200),
        training=TrainingConfig(local_batch_size=1, seq_len=8192, steps=1000, mixed_precision_param="bfloat16",
                                mixed_precision_reduce="float32", dtype="bfloat16"),
        dataloader=SyntheticDataLoaderConfig(seed=0),
        # sharded runs keep the gathered bf16 weights (16 GB) between forward and backward: one all-gather per layer
        # and step instead of two (+1.4 % tokens/s on 8 GPUs)
        parallelism=ParallelismConfig(data_parallel_shard_degree=-1, fsdp_reshard_after_forward="never"),
        checkpoint=CheckpointConfig(interval=500),
        # selective checkpointing with the rule that keeps every contraction (GEMM, attention) and recomputes norms,
        # rotary embedding, SwiGLU and residual adds: about 2 % of the step for 9 GB.  `llama3_8b_noac` drops it (an 8B
        # model at seq 8192 peaks at 112 GB on ONE 180 GB GPU, 96 GB of it weights, gradients and fp32 AdamW state).
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="op_save_all_mm",
                                                         selective_keep_swiglu=True),
        # every operator of the block that this framework owns: norms, rotary embedding, SwiGLU, the loss and all
        # projections (tcgen05 GEMMs); attention stays on the fused library kernel
        model_converters=ModelConvertersConfig(
            converters=[*_fused_converters(), get_model_converter_config("b200_linear")]),
    )


def llama3_8b_noac() -> TrainerConfig:
    """`llama3_8b` without activation checkpointing (fits a 180 GB GPU even unsharded)."""
    cfg = llama3_8b()
    cfg.activation_checkpoint.mode = "none"
    return cfg


def llama3_8b_mxfp8() -> TrainerConfig:
    """`llama3_8b` with every attention and feed-forward projection in MXFP8 (block-scaled tensor-core GEMMs for
    forward, input gradient and weight gradient; fp8 saved activations); embeddings, norms and the output head stay
    bf16."""
    from titan_b200.lowp.mx_converter import MXFP8Converter

    cfg = llama3_8b()
    # measured without recomputation (111 GB on one GPU): the fp8 copies the MX linears keep are half the size of the
    # bf16 activations they replace.  Selective checkpointing works too (`titan_b200::mx_linear_fwd` is on its save
    # list, so a checkpointed block does not quantise and multiply twice).
    cfg.activation_checkpoint.mode = "none"
    cfg.model_converters.converters.append(
        MXFP8Converter.Config(recipe_name="mxfp8_rceil", fqns=["attention.w", "feed_forward.w"]))
    return cfg


def llama3_8b_baseline() -> TrainerConfig:
    """Same model, shapes, checkpointing rule and FSDP reshard policy as `llama3_8b` on library ops only (cuBLAS,
    cuDNN SDPA, torch fused AdamW, NCCL collectives issued by FSDP2): the on-box comparator."""
    cfg = llama3_8b()
    cfg.model_converters = ModelConvertersConfig(converters=[])
    cfg.optimizer.implementation = "fused"
    cfg.parallelism.fsdp_fused_collectives = False
    return cfg


def llama3_8b_baseline_upstream_ac() -> TrainerConfig:
    """`llama3_8b_baseline` with the upstream selective rule (every second matmul recomputed) and upstream's
    reshard-after-forward default."""
    cfg = llama3_8b_baseline()
    cfg.activation_checkpoint.selective_ac_option = "op"
    cfg.parallelism.fsdp_reshard_after_forward = "default"
    return cfg


def llama3_70b() -> TrainerConfig:
    """Llama-3 70B: FSDP=4 × TP=2 with sequence parallel, full AC, Swap Optimizer (AdamW state in pinned host memory)."""
    return TrainerConfig(
        model=ModelConfigRef(name="llama3", flavor="70B"),
        metrics=MetricsConfig(log_freq=10),
        optimizer=OptimizerConfig(name="AdamW", lr=1.5e-4, eps=1e-8, swap_optimizer=True, swap_optimizer_times=16),
        lr_scheduler=LRSchedulerConfig(warmup_steps=200),
        training=TrainingConfig(local_batch_size=1, seq_len=8192, steps=1000, mixed_precision_param="bfloat16",
                                mixed_precision_reduce="float32", dtype="bfloat16"),
        dataloader=SyntheticDataLoaderConfig(seed=0),
        parallelism=ParallelismConfig(data_parallel_shard_degree=-1, tensor_parallel_degree=2,
                                      enable_async_tensor_parallel=True),
        checkpoint=CheckpointConfig(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
        model_converters=ModelConvertersConfig(converters=_fused_converters()),
    )


def llama3_405b() -> TrainerConfig:
    cfg = llama3_70b()
    cfg.model = ModelConfigRef(name="llama3", flavor="405B")
    cfg.parallelism.tensor_parallel_degree = 8
    cfg.optimizer.lr = 8e-5
    return cfg
