"""DeepSeek-V3 recipes (``--module deepseek_v3 --config <name>``).

Mirrors the reference's recipe set (torchtitan_npu/models/deepseek_v3/config_registry.py:35-258) and adds
the 16B EP=8 MXFP8 recipe of the B200 benchmark suite.
"""

from dataclasses import replace

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
    debug_single_node_eq_pruned_config,
    trainer_base_config,
)
from titan_b200.protocols.converter import get_model_converter_config


def _converters(*names):
    return ModelConvertersConfig(converters=[get_model_converter_config(n) for n in names])


_MOE_FUSED = ("b200_rms_norm", "b200_rope", "b200_moe_dispatch", "b200_gmm")


def deepseek_v3_debugmodel() -> TrainerConfig:
    return TrainerConfig(
        model=ModelConfigRef(name="deepseek_v3", flavor="debugmodel"),
        metrics=MetricsConfig(log_freq=1),
        optimizer=OptimizerConfig(lr=8e-4, implementation="for-loop"),
        lr_scheduler=LRSchedulerConfig(warmup_steps=2, decay_ratio=0.8),
        training=TrainingConfig(local_batch_size=2, seq_len=256, steps=10, mixed_precision_param="float32",
                                dtype="float32"),
        dataloader=SyntheticDataLoaderConfig(seed=0),
        activation_checkpoint=ActivationCheckpointConfig(mode="none"),
    )


def deepseek_v3_smoketest() -> TrainerConfig:
    """dim 128, 4 layers, 8 experts: 2 steps, selective AC."""
    cfg = deepseek_v3_debugmodel()
    cfg.model = ModelConfigRef(name="deepseek_v3", flavor="smoketest")
    cfg.training = replace(cfg.training, steps=2, seq_len=128)
    cfg.activation_checkpoint = ActivationCheckpointConfig(mode="selective", selective_ac_option="op")
    return cfg


def deepseek_v3_671b_debug() -> TrainerConfig:
    """Pruned 671B (dim 7168, 4 layers, 8 experts): TP2 EP2, swap optimizer, full AC, seq 2048, local batch 2."""
    base = debug_single_node_eq_pruned_config(trainer_base_config())
    return replace(
        base,
        model=ModelConfigRef(name="deepseek_v3", flavor="671B_debug"),
        training=replace(base.training, local_batch_size=2, seq_len=2048, dtype="bfloat16"),
        parallelism=replace(base.parallelism, tensor_parallel_degree=2, expert_parallel_degree=2,
                            expert_tensor_parallel_degree=1),
        dataloader=SyntheticDataLoaderConfig(seed=0),
        model_converters=_converters(*_MOE_FUSED),
    )


def deepseek_v3_671b_16die_debug() -> TrainerConfig:
    """Same pruned model with TP2 × PP4 (1F1B) × EP4, seq 4096, local batch 4."""
    base = deepseek_v3_671b_debug()
    return replace(
        base,
        training=replace(base.training, local_batch_size=4, seq_len=4096),
        parallelism=replace(base.parallelism, tensor_parallel_degree=2, pipeline_parallel_degree=4,
                            pipeline_parallel_schedule="1F1B", expert_parallel_degree=4),
    )


def deepseek_v3_671b_61layers_4k() -> TrainerConfig:
    """Full 61-layer model: TP4 EP128, global batch 1024, seq 4096 (a 128-rank job)."""
    base = trainer_base_config()
    return replace(
        base,
        model=ModelConfigRef(name="deepseek_v3", flavor="671B"),
        training=replace(base.training, local_batch_size=1, global_batch_size=1024, seq_len=4096, dtype="bfloat16"),
        parallelism=replace(base.parallelism, tensor_parallel_degree=4, expert_parallel_degree=128,
                            expert_tensor_parallel_degree=1),
        debug=replace(base.debug, moe_force_load_balance=True),
        model_converters=_converters(*_MOE_FUSED),
    )


def deepseek_v3_16b_ep8() -> TrainerConfig:
    """DeepSeek-V3-style 16B MoE with true MLA dims: EP=8 + FSDP on 8 GPUs, bf16, seq 4096, local batch 2."""
    return TrainerConfig(
        model=ModelConfigRef(name="deepseek_v3", flavor="16B_mla"),
        metrics=MetricsConfig(log_freq=10),
        optimizer=OptimizerConfig(lr=2.2e-4, eps=1e-8, implementation="b200_fused"),
        lr_scheduler=LRSchedulerConfig(warmup_steps=200, decay_ratio=0.8, decay_type="cosine", min_lr_factor=0.1),
        training=TrainingConfig(local_batch_size=2, seq_len=4096, steps=1000, dtype="bfloat16"),
        dataloader=SyntheticDataLoaderConfig(seed=0),
        parallelism=ParallelismConfig(expert_parallel_degree=8, expert_parallel_comm_backend="fused_p2p"),
        checkpoint=CheckpointConfig(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="op"),
        model_converters=_converters(*_MOE_FUSED),
    )


def deepseek_v3_16b_ep8_mxfp8() -> TrainerConfig:
    """As above with MXFP8 (1x32 e8m0 block scales, e4m3) expert GEMMs; must come after the grouped-GEMM converter."""
    from titan_b200.lowp.mx_converter import MXFP8Converter

    cfg = deepseek_v3_16b_ep8()
    cfg.model_converters.converters.append(MXFP8Converter.Config(recipe_name="mxfp8_rceil", fqns=["moe.experts"]))
    return cfg
