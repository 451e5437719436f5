"""VLM recipes (reference: torchtitan_npu/models/vlm/config_registry.py:30-77)."""

from dataclasses import replace

from titan_b200.config.configs import (
    ActivationCheckpointConfig,
    CheckpointConfig,
    CompileConfig,
    LRSchedulerConfig,
    MetricsConfig,
    ModelConfigRef,
    ModelConvertersConfig,
    MultiModalDataLoaderConfig,
    OptimizerConfig,
    ParallelismConfig,
    ProfilingConfig,
    TrainerConfig,
    TrainingConfig,
)
from titan_b200.protocols.converter import get_model_converter_config

VLM_TOKENIZER_ASSETS_PATH = "./tests/assets/tokenizer/vlm_tokenizer"


def vlm_debugmodel() -> TrainerConfig:
    return TrainerConfig(
        model=ModelConfigRef(name="vlm", flavor="debugmodel", hf_assets_path=VLM_TOKENIZER_ASSETS_PATH),
        model_converters=ModelConvertersConfig(converters=[get_model_converter_config("b200_vlm")]),
        metrics=MetricsConfig(log_freq=1),
        dataloader=MultiModalDataLoaderConfig(dataset="synthetic", max_patches_per_image=1024,
                                              max_images_per_batch=64),
        optimizer=OptimizerConfig(name="AdamW", lr=8e-4, implementation="for-loop"),
        lr_scheduler=LRSchedulerConfig(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0),
        training=TrainingConfig(local_batch_size=8, seq_len=2048, steps=10),
        parallelism=ParallelismConfig(data_parallel_replicate_degree=1, data_parallel_shard_degree=-1,
                                      tensor_parallel_degree=1, context_parallel_degree=1,
                                      pipeline_parallel_degree=1, fsdp_reshard_after_forward="always"),
        checkpoint=CheckpointConfig(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="none"),
        profiling=ProfilingConfig(enable_profiling=False),
    )


def vlm_debugmodel_compile() -> TrainerConfig:
    return replace(vlm_debugmodel(), compile=CompileConfig(enable=True))
