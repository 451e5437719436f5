#!/usr/bin/env bash
# Continued pre-training of DeepSeek-V4 Flash (43 layers, 256 experts) at seq 4096 from Hugging Face weights, on
# NNODES nodes of 8 B200s.  Run on every node with the same NODE_IPS list; the node's own address picks its rank.
#
#   NODE_IPS="10.0.0.1 10.0.0.2 ..." HF_CKPT=/ckpt/deepseek-v4-flash ./examples/deepseek_v4/cpt_deepseek_v4_flash_4k.sh
set -euo pipefail
cd "$(dirname "$0")/../.."
: "${HF_CKPT:?set HF_CKPT to the folder with the Hugging Face safetensors}"
MODULE=deepseek_v4 CONFIG=deepseek_v4_flash_4k_128die ./scripts/run_train_multinodes.sh \
    --checkpoint.initial_load_path "${HF_CKPT}" --checkpoint.initial_load_in_hf --checkpoint.initial_load_model_only \
    --training.seq_len 4096 --training.num_mtp_modules 1 "$@"
