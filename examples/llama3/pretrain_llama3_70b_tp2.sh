#!/usr/bin/env bash
# Llama-3 70B on one node: tensor parallel 2 with the all-gather / reduce-scatter of sequence parallelism fused into
# the projection GEMMs (async TP over peer memory), FSDP over the remaining 4-way data-parallel dimension.
set -euo pipefail
cd "$(dirname "$0")/../.."
NGPU=${NGPU:-8} MODULE=llama3 CONFIG=llama3_70b ./scripts/run_train.sh \
    --parallelism.tensor_parallel_degree 2 --parallelism.enable_async_tensor_parallel \
    --training.local_batch_size 1 --training.seq_len 8192 "$@"
