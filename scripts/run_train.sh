#!/usr/bin/env bash
# Single-node launcher: one process per GPU over NCCL.
#
#   NGPU=8 MODULE=llama3 CONFIG=llama3_8b ./scripts/run_train.sh --training.steps 100
#   COMM_MODE=fake_backend NGPU=64 MODULE=deepseek_v3 CONFIG=... ./scripts/run_train.sh     # one-process dry run
#
# Everything after the script name goes to the trainer as --section.field overrides.
# (reference: scripts/run_train.sh:13-40)
set -euo pipefail

NGPU=${NGPU:-8}
export LOG_RANK=${LOG_RANK:-0}
MODULE=${MODULE:-qwen3}
CONFIG=${CONFIG:-debug_qwen3_06b_single_node}
TRAIN_FILE=${TRAIN_FILE:-titan_b200.entry}
COMM_MODE=${COMM_MODE:-}
MASTER_PORT=${MASTER_PORT:-29500}

cd "$(dirname "$0")/.."

if [ -n "${COMM_MODE}" ]; then
    echo "Running with comm_mode=${COMM_MODE}"
    NGPU="${NGPU}" LOCAL_RANK=0 python -m "${TRAIN_FILE}" \
        --module "${MODULE}" --config "${CONFIG}" \
        --comm.mode="${COMM_MODE}" --training.steps=1 "$@"
else
    # expandable segments keep the caching allocator from fragmenting under FSDP's gather/free pattern;
    # one connection per device keeps kernel launch order = stream order for comm/compute overlap
    PYTORCH_CUDA_ALLOC_CONF="expandable_segments:True" \
    CUDA_DEVICE_MAX_CONNECTIONS=${CUDA_DEVICE_MAX_CONNECTIONS:-1} \
    TORCH_NCCL_AVOID_RECORD_STREAMS=1 \
    python -m torch.distributed.run --nnodes=1 --nproc-per-node="${NGPU}" \
        --master-addr 127.0.0.1 --master-port "${MASTER_PORT}" \
        --local-ranks-filter "${LOG_RANK}" --role rank --tee 3 \
        -m "${TRAIN_FILE}" --module "${MODULE}" --config "${CONFIG}" "$@"
fi
