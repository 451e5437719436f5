"""DeepSeek-V4 recipes (reference: torchtitan_npu/models/deepseek_v4/config_registry.py:22-121)."""

from dataclasses import replace

from titan_b200.config.configs import (
    ActivationCheckpointConfig,
    LRSchedulerConfig,
    MetricsConfig,
    ModelConfigRef,
    ModelConvertersConfig,
    OptimizerConfig,
    SyntheticDataLoaderConfig,
    TrainerConfig,
    TrainingConfig,
    cpt_default_config,
    debug_single_node_eq_pruned_config,
    trainer_base_config,
)
from titan_b200.protocols.converter import get_model_converter_config

# linears that run in MXFP8 in the low-precision recipes
_MXFP8_FQNS = ("pre_attention.wq_a", "pre_attention.wq_b", "pre_attention.wkv", "pre_attention.indexer.wq_b",
               "pre_attention.indexer.weights_proj", "post_attention.wo_a", "post_attention.wo_b", "moe.experts",
               "moe.shared_experts", "e_proj", "h_proj")
_DEFAULT = ("b200_rms_norm", "b200_moe_dispatch", "b200_gmm", "b200_rope", "b200_smla", "b200_mhc_pre")


def _converters(*names):
    return ModelConvertersConfig(converters=[get_model_converter_config(n) for n in names])


def deepseek_v4_smoketest() -> TrainerConfig:
    """CPU-sized model: 4 layers covering ratios 1 / 4 / 128, hash routing in layer 0, one MTP depth."""
    return TrainerConfig(
        model=ModelConfigRef(name="deepseek_v4", flavor="smoketest"),
        metrics=MetricsConfig(log_freq=1),
        optimizer=OptimizerConfig(lr=8e-4, implementation="for-loop"),
        lr_scheduler=LRSchedulerConfig(warmup_steps=2),
        training=TrainingConfig(local_batch_size=2, seq_len=256, steps=2, mixed_precision_param="float32",
                                dtype="float32", num_mtp_modules=1),
        dataloader=SyntheticDataLoaderConfig(seed=0),
        activation_checkpoint=ActivationCheckpointConfig(mode="none"),
    )


def debug_deepseek_v4_single_node_1b() -> TrainerConfig:
    base = trainer_base_config()
    return replace(
        base,
        model=ModelConfigRef(name="deepseek_v4", flavor="mini_1b"),
        model_converters=_converters("b200_rms_norm", "b200_moe_dispatch", "b200_gmm", "b200_rope"),
        optimizer=replace(base.optimizer, swap_optimizer=False),
        lr_scheduler=replace(base.lr_scheduler, min_lr_factor=0.1, warmup_steps=2),
        training=replace(base.training, seq_len=576, steps=2, num_mtp_modules=0),
        dataloader=SyntheticDataLoaderConfig(seed=0),
        activation_checkpoint=replace(base.activation_checkpoint, mode="none"),
    )


def _flash_base() -> TrainerConfig:
    base = trainer_base_config()
    return replace(base, model=ModelConfigRef(name="deepseek_v4", flavor="v4_flash_43layers_256experts"),
                   model_converters=_converters(*_DEFAULT), training=replace(base.training, num_mtp_modules=1))


def deepseek_v4_flash_4k_128die() -> TrainerConfig:
    base = cpt_default_config(_flash_base())
    return replace(base, training=replace(base.training, global_batch_size=1024),
                   parallelism=replace(base.parallelism, data_parallel_shard_degree=128, expert_parallel_degree=64))


def deepseek_v4_pro_4k_384die() -> TrainerConfig:
    base = deepseek_v4_flash_4k_128die()
    return replace(base, model=ModelConfigRef(name="deepseek_v4", flavor="v4_pro_61layers_384experts"),
                   training=replace(base.training, global_batch_size=384),
                   parallelism=replace(base.parallelism, data_parallel_shard_degree=384, expert_parallel_degree=192))


def debug_deepseek_v4_flash_single_node() -> TrainerConfig:
    base = debug_single_node_eq_pruned_config(_flash_base())
    return replace(base, model=ModelConfigRef(name="deepseek_v4", flavor="v4_flash_43layers_16experts"),
                   model_converters=_converters(*_DEFAULT, "b200_mhc_post"),
                   dataloader=SyntheticDataLoaderConfig(seed=0),
                   parallelism=replace(base.parallelism, expert_parallel_degree=8))


def debug_deepseek_v4_flash_single_node_mxfp8() -> TrainerConfig:
    from titan_b200.lowp.mx_converter import MXFP8ConverterConfig

    base = debug_deepseek_v4_flash_single_node()
    convs = list(base.model_converters.converters) + [
        MXFP8ConverterConfig(recipe_name="mxfp8_rceil", fqns=list(_MXFP8_FQNS))]
    return replace(base, model_converters=ModelConvertersConfig(converters=convs))


def debug_deepseek_v4_pro_single_node() -> TrainerConfig:
    base = debug_deepseek_v4_flash_single_node()
    return replace(base, model=ModelConfigRef(name="deepseek_v4", flavor="v4_pro_16layers_16experts"),
                   model_converters=_converters(*_DEFAULT),
                   parallelism=replace(base.parallelism, expert_parallel_degree=16))
