"""Qwen3 recipes (reference: torchtitan_npu/models/qwen3/config_registry.py:23-142)."""

from dataclasses import replace

from titan_b200.config.configs import (
    ChatDataLoaderConfig,
    ModelConfigRef,
    ModelConvertersConfig,
    SyntheticDataLoaderConfig,
    TrainerConfig,
    debug_single_node_eq_pruned_config,
    sft_default_config,
    trainer_base_config,
)
from titan_b200.models.qwen3.tnd_config import enable_varlen_attention
from titan_b200.protocols.converter import get_model_converter_config

_DEFAULT = ("b200_rms_norm", "b200_rope", "b200_moe_dispatch", "b200_gmm")


def _converters(*names):
    return ModelConvertersConfig(converters=[get_model_converter_config(n) for n in names])


def qwen3_debugmodel() -> TrainerConfig:
    base = trainer_base_config()
    return replace(base, model=ModelConfigRef(name="qwen3", flavor="debugmodel"),
                   training=replace(base.training, local_batch_size=2, seq_len=256, steps=5, dtype="float32",
                                    mixed_precision_param="float32"),
                   optimizer=replace(base.optimizer, swap_optimizer=False, implementation="for-loop"),
                   dataloader=SyntheticDataLoaderConfig(seed=0),
                   activation_checkpoint=replace(base.activation_checkpoint, mode="none"))


def qwen3_debugmodel_moe() -> TrainerConfig:
    base = qwen3_debugmodel()
    return replace(base, model=ModelConfigRef(name="qwen3", flavor="debugmodel_moe"))


def _qwen3_06b_base() -> TrainerConfig:
    base = trainer_base_config()
    return replace(base, model=ModelConfigRef(name="qwen3", flavor="0.6B",
                                              hf_assets_path="./tests/assets/tokenizer/qwen3-tokenizer"),
                   model_converters=ModelConvertersConfig(converters=[]))


def debug_qwen3_06b_single_node() -> TrainerConfig:
    base = debug_single_node_eq_pruned_config(_qwen3_06b_base())
    return replace(base, dataloader=SyntheticDataLoaderConfig(seed=0),
                   checkpoint=replace(base.checkpoint, load_only=False))


def _qwen3_30ba3b_base() -> TrainerConfig:
    base = trainer_base_config()
    return replace(base, model=ModelConfigRef(name="qwen3", flavor="30B-A3B", hf_assets_path="./assets/hf/Qwen3-30B-A3B"),
                   model_converters=_converters(*_DEFAULT))


def sft_qwen3_30ba3b_gsm8k() -> TrainerConfig:
    """GSM8K SFT of the 30B-A3B MoE: EP8 × Ulysses CP4, selective AC, HF initial load."""
    base = sft_default_config(_qwen3_30ba3b_base())
    return replace(
        base,
        optimizer=replace(base.optimizer, lr=1e-5),
        lr_scheduler=replace(base.lr_scheduler, warmup_steps=10, decay_ratio=0.9, min_lr_factor=0.1),
        training=replace(base.training, local_batch_size=1, seq_len=4096, steps=100),
        parallelism=replace(base.parallelism, expert_parallel_degree=8, context_parallel_degree=4),
        dataloader=ChatDataLoaderConfig(dataset_path="openai/gsm8k",
                                        load_dataset_kwargs={"name": "main", "split": "train"},
                                        chat_processor="titan_b200.data.chat_processors:process_gsm8k_sample"),
        checkpoint=replace(base.checkpoint, enable=True, initial_load_in_hf=True,
                           initial_load_path="./assets/hf/Qwen3-30B-A3B"),
        activation_checkpoint=replace(base.activation_checkpoint, mode="selective"),
    )


def sft_qwen3_30ba3b_gsm8k_tnd() -> TrainerConfig:
    """The GSM8K recipe with packed variable-length attention (documents do not attend to each other)."""
    base = sft_qwen3_30ba3b_gsm8k()
    return replace(base, model=enable_varlen_attention(base.model))


def _qwen3_1_7b_base() -> TrainerConfig:
    base = trainer_base_config()
    return replace(base, model=ModelConfigRef(name="qwen3", flavor="1.7B", hf_assets_path="./assets/hf/Qwen3-1.7B"),
                   model_converters=ModelConvertersConfig(converters=[]))


def sft_qwen3_1_7b_wordle() -> TrainerConfig:
    """20-step SFT warm-up of Qwen3-1.7B on multi-turn Wordle transcripts, from the HF base weights, one GPU."""
    base = sft_default_config(_qwen3_1_7b_base())
    return replace(
        base,
        optimizer=replace(base.optimizer, lr=1e-5),
        lr_scheduler=replace(base.lr_scheduler, warmup_steps=0, decay_ratio=1.0, min_lr_factor=1.0),
        training=replace(base.training, local_batch_size=2, global_batch_size=64, seq_len=1024, max_norm=1.0,
                         steps=20),
        dataloader=ChatDataLoaderConfig(dataset_path="willcb/V3-wordle", load_dataset_kwargs={"split": "train"},
                                        chat_processor="titan_b200.data.chat_processors:process_wordle_sample"),
        checkpoint=replace(base.checkpoint, folder="checkpoint_wordle_sft", initial_load_in_hf=True,
                           initial_load_path="./assets/hf/Qwen3-1.7B"),
        activation_checkpoint=replace(base.activation_checkpoint, mode="selective"),
        profiling=replace(base.profiling, profile_ranks=[0], profile_step_start=6, profile_step_end=7,
                          profile_with_memory=True),
    )
