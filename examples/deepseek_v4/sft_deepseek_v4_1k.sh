#!/usr/bin/env bash
# Supervised fine-tuning of the 1B-class DeepSeek-V4 on a chat dataset at seq 1152 (a multiple of the compressor's
# 128-token ratio): weights from a Hugging Face folder, DSV4 chat encoding, loss on assistant tokens only, conversations
# packed into fixed-length rows, bf16 export of the last checkpoint.
#
#   HF_ASSETS_PATH=/models/deepseek-v4-mini-1B DATA_FILES=yelp_review_full/train-00000-of-00001.parquet \
#       ./examples/deepseek_v4/sft_deepseek_v4_1k.sh
set -euo pipefail
cd "$(dirname "$0")/../.."
HF_ASSETS_PATH=${HF_ASSETS_PATH:?folder with tokenizer.json and the safetensors}
DATA_FILES=${DATA_FILES:?parquet / jsonl file(s) of the chat dataset}
[ -f "${HF_ASSETS_PATH}/tokenizer.json" ] || { echo "no tokenizer.json under ${HF_ASSETS_PATH}" >&2; exit 1; }
NGPU=${NGPU:-8} MODULE=deepseek_v4 CONFIG=${CONFIG:-debug_deepseek_v4_single_node_1b} ./scripts/run_train.sh \
    --model.hf_assets_path "${HF_ASSETS_PATH}" \
    --checkpoint.enable --checkpoint.initial_load_path "${CHECKPOINT_INITIAL_LOAD_PATH:-${HF_ASSETS_PATH}}" \
    --checkpoint.initial_load_in_hf --checkpoint.initial_load_model_only \
    --checkpoint.folder "${CHECKPOINT_FOLDER:-checkpoint}" --checkpoint.interval 500 \
    --checkpoint.last_save_model_only --checkpoint.export_dtype bfloat16 \
    --training.local_batch_size 8 --training.seq_len 1152 --training.steps 1000 --lr_scheduler.warmup_steps 60 \
    "$@" \
    dataloader:chat_data_loader_config \
    --dataloader.dataset_path parquet --dataloader.data_files "${DATA_FILES}" \
    --dataloader.dataset_split "${DATASET_SPLIT:-train}" \
    --dataloader.chat_processor titan_b200.data.chat_processors.process_yelp_sample \
    dataloader.chat_encoder:dsv4_encoder_config
