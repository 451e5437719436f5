#!/usr/bin/env bash
# Continued pre-training of DeepSeek-V4 Pro (61 layers, 384 experts) at seq 4096 from Hugging Face weights.
set -euo pipefail
cd "$(dirname "$0")/../.."
: "${HF_CKPT:?set HF_CKPT to the folder with the Hugging Face safetensors}"
MODULE=deepseek_v4 CONFIG=deepseek_v4_pro_4k_384die ./scripts/run_train_multinodes.sh \
    --checkpoint.initial_load_path "${HF_CKPT}" --checkpoint.initial_load_in_hf --checkpoint.initial_load_model_only \
    --training.seq_len 4096 "$@"
