#!/usr/bin/env bash
# Qwen3-30B-A3B SFT on GSM8K: expert parallel 8, Ulysses context parallel 4, ChatML encoding.
# `CONFIG=sft_qwen3_30ba3b_gsm8k_tnd` packs conversations and attends per document (varlen attention).
set -euo pipefail
cd "$(dirname "$0")/../.."
NGPU=${NGPU:-8} MODULE=qwen3 CONFIG=${CONFIG:-sft_qwen3_30ba3b_gsm8k} ./scripts/run_train.sh "$@"
