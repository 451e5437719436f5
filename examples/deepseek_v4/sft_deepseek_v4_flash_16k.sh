#!/usr/bin/env bash
# Long-context SFT of DeepSeek-V4 Flash at seq 16384 on several nodes: context parallel 4 (the compressor / indexer
# attention exchanges its window and compressed keys between sequence shards) on top of the recipe's FSDP x EP layout,
# packed conversations.  Run on every node with the same NODE_IPS list.
set -euo pipefail
cd "$(dirname "$0")/../.."
HF_ASSETS_PATH=${HF_ASSETS_PATH:?folder with tokenizer.json and the safetensors}
DATA_FILES=${DATA_FILES:?parquet / jsonl file(s) of the chat dataset}
MODULE=deepseek_v4 CONFIG=deepseek_v4_flash_4k_128die ./scripts/run_train_multinodes.sh \
    --model.hf_assets_path "${HF_ASSETS_PATH}" \
    --checkpoint.enable --checkpoint.initial_load_path "${HF_ASSETS_PATH}" --checkpoint.initial_load_in_hf \
    --training.seq_len 16384 --training.local_batch_size 1 --parallelism.context_parallel_degree 4 \
    --optimizer.lr 5e-6 --lr_scheduler.warmup_steps 30 \
    "$@" \
    dataloader:chat_data_loader_config \
    --dataloader.dataset_path parquet --dataloader.data_files "${DATA_FILES}" \
    --dataloader.chat_processor titan_b200.data.chat_processors.process_yelp_sample \
    dataloader.chat_encoder:dsv4_encoder_config
