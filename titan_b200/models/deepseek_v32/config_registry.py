"""DeepSeek-V3.2 recipes (reference: torchtitan_npu/models/deepseek_v32/config_registry.py:36-208)."""

from dataclasses import replace

from titan_b200.config.configs import (
    ActivationCheckpointConfig,
    LRSchedulerConfig,
    MetricsConfig,
    ModelConfigRef,
    ModelConvertersConfig,
    OptimizerConfig,
    ParallelismConfig,
    SyntheticDataLoaderConfig,
    TrainerConfig,
    TrainingConfig,
    debug_single_node_eq_pruned_config,
    trainer_base_config,
)
from titan_b200.protocols.converter import get_model_converter_config

_FUSED = ("b200_dsa", "b200_rms_norm", "b200_rope", "b200_moe_dispatch", "b200_gmm")


def _converters(*names):
    return ModelConvertersConfig(converters=[get_model_converter_config(n) for n in names])


def deepseek_v32_smoketest() -> TrainerConfig:
    return TrainerConfig(
        model=ModelConfigRef(name="deepseek_v32", flavor="smoketest"),
        metrics=MetricsConfig(log_freq=1),
        optimizer=OptimizerConfig(lr=8e-4, implementation="for-loop"),
        lr_scheduler=LRSchedulerConfig(warmup_steps=2),
        training=TrainingConfig(local_batch_size=2, seq_len=128, steps=2, mixed_precision_param="float32",
                                dtype="float32"),
        dataloader=SyntheticDataLoaderConfig(seed=0),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="op"),
    )


def deepseek_v32_671b_4layers_debug() -> TrainerConfig:
    """Pruned 671B (4 layers, 16 experts): EP8, swap optimizer, full AC."""
    base = debug_single_node_eq_pruned_config(trainer_base_config())
    return replace(
        base,
        model=ModelConfigRef(name="deepseek_v32", flavor="671B_debug_4_layers"),
        training=replace(base.training, local_batch_size=1, seq_len=4096, dtype="bfloat16"),
        parallelism=replace(base.parallelism, expert_parallel_degree=8),
        dataloader=SyntheticDataLoaderConfig(seed=0),
        model_converters=_converters(*_FUSED),
    )


def deepseek_v32_671b_61layers_4k() -> TrainerConfig:
    base = trainer_base_config()
    return replace(
        base,
        model=ModelConfigRef(name="deepseek_v32", flavor="671B"),
        training=replace(base.training, local_batch_size=1, global_batch_size=512, seq_len=4096, dtype="bfloat16"),
        parallelism=replace(base.parallelism, tensor_parallel_degree=4, expert_parallel_degree=64),
        debug=replace(base.debug, moe_force_load_balance=True),
        model_converters=_converters(*_FUSED),
    )


def deepseek_v32_671b_61layers_32k() -> TrainerConfig:
    """Long context: TP4 EP64 CP8, seq 32768, global batch 128."""
    cfg = deepseek_v32_671b_61layers_4k()
    return replace(
        cfg,
        training=replace(cfg.training, seq_len=32768, global_batch_size=128),
        parallelism=replace(cfg.parallelism, context_parallel_degree=8),
    )


def deepseek_v32_sparse_cp8() -> TrainerConfig:
    """12-layer sparse-attention model at seq 131072 on 8 GPUs: CP=8 (DSA all-gather of the shared KV latent),
    lightning indexer scored in bf16 on the tensor cores, top-2048 keys per query."""
    return TrainerConfig(
        model=ModelConfigRef(name="deepseek_v32", flavor="sparse_12l"),
        metrics=MetricsConfig(log_freq=1),
        optimizer=OptimizerConfig(lr=1e-4, implementation="b200_fused"),
        lr_scheduler=LRSchedulerConfig(warmup_steps=20),
        training=TrainingConfig(local_batch_size=1, seq_len=131072, steps=100, dtype="bfloat16"),
        dataloader=SyntheticDataLoaderConfig(seed=0),
        parallelism=ParallelismConfig(context_parallel_degree=8, data_parallel_shard_degree=1),
        # keep what is expensive to recompute and small to store (contraction outputs, the indexer's selection, the
        # sparse-attention output); recompute the elementwise rest
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="op_save_all_mm"),
        model_converters=_converters(*_FUSED),
    )
