#!/usr/bin/env bash
# Llama-3 8B pre-training, seq 8192, one node of B200s: FSDP over all GPUs, fused kernels, no activation recomputation
# (the 8B model at this sequence length fits a 180 GB GPU without it).
#
#   NGPU=8 ./examples/llama3/pretrain_llama3_8b.sh --training.steps 1000 \
#       dataloader:text_data_loader_config --dataloader.dataset c4 --dataloader.dataset_path /data/c4
# (the recipe trains on synthetic tokens unless the data loader is switched as above)
#
# Measured on B200: 20.1k tokens/s on one GPU, 148.8k tokens/s on eight.
set -euo pipefail
cd "$(dirname "$0")/../.."
NGPU=${NGPU:-8} MODULE=llama3 CONFIG=llama3_8b ./scripts/run_train.sh \
    --training.local_batch_size 1 --training.seq_len 8192 \
    --metrics.log_freq 10 "$@"
