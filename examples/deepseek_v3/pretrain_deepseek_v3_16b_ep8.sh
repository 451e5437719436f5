#!/usr/bin/env bash
# DeepSeek-V3 16B (MLA, 64 routed experts, top-6) on one node: expert parallel 8 inside FSDP 8.  The MoE layers use the
# fused peer-memory dispatch / combine (token rows are put straight into the owner's expert-major buffer over NVLink)
# and the grouped tcgen05 GEMM.  `CONFIG=deepseek_v3_16b_ep8_mxfp8` runs the experts and attention projections in MXFP8.
#
# Measured on 8 B200s with forced load balance: 148k tokens/s fused vs 129k through NCCL all-to-all.
set -euo pipefail
cd "$(dirname "$0")/../.."
NGPU=${NGPU:-8} MODULE=deepseek_v3 CONFIG=${CONFIG:-deepseek_v3_16b_ep8} ./scripts/run_train.sh \
    --parallelism.expert_parallel_degree 8 --parallelism.expert_parallel_capacity_factor 4.0 "$@"
