#!/usr/bin/env bash
# Multi-node launcher: run the same command on every node.
#
#   NODE_IPS=10.0.0.1,10.0.0.2 NGPU=8 MODULE=deepseek_v32 CONFIG=deepseek_v32_671b_61layers_4k \
#       ./scripts/run_train_multinodes.sh [--section.field value ...]
#
# The node rank is the position of this host's address in NODE_IPS (or NODE_RANK when set); the first address is the
# rendezvous master.  Logs are tee'd to logs/<config>_<time>_node<rank>.log.  The script starts nothing else and stops
# nothing: a stale job has to be ended by its owner through its own process group.
# (reference: scripts/run_train_multinodes.sh:20-75)
set -euo pipefail

# COMM_MODE=fake_backend: one process, no rendezvous: builds the model for the full world size and runs one step on
# fake collectives (a dry run of the recipe and of the command line).
if [ -n "${COMM_MODE:-}" ]; then
    cd "$(dirname "$0")/.."
    NGPU="${NGPU:-8}" LOCAL_RANK=0 exec python -m "${TRAIN_FILE:-titan_b200.entry}" \
        --module "${MODULE:-deepseek_v32}" --config "${CONFIG:-deepseek_v32_671b_61layers_4k}" \
        --comm.mode="${COMM_MODE}" --training.steps=1 "$@"
fi

if command -v ip > /dev/null 2>&1; then
    export NCCL_SOCKET_IFNAME=${NCCL_SOCKET_IFNAME:-$(ip -o -4 addr show scope global | awk '$2 != "docker0" {print $2; exit}')}
    LOCAL_HOST=${LOCAL_HOST:-$(ip addr show "${NCCL_SOCKET_IFNAME}" | grep "inet " | awk '{print $2}' | cut -d'/' -f1 | head -n1)}
fi
[ -n "${NCCL_SOCKET_IFNAME:-}" ] && export GLOO_SOCKET_IFNAME=${GLOO_SOCKET_IFNAME:-${NCCL_SOCKET_IFNAME}}
export PYTORCH_CUDA_ALLOC_CONF=${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}
export CUDA_DEVICE_MAX_CONNECTIONS=${CUDA_DEVICE_MAX_CONNECTIONS:-1}
export TORCH_NCCL_AVOID_RECORD_STREAMS=1
export LOG_RANK=${LOG_RANK:-0}
export PYTHONUNBUFFERED=1

LOCAL_HOST=${LOCAL_HOST:-$(hostname -I 2> /dev/null | awk '{print $1}')}
LOCAL_HOST=${LOCAL_HOST:-127.0.0.1}
if [[ -n "${NODE_IPS:-}" ]]; then
    read -r -a IPs <<< "${NODE_IPS//,/ }"
else
    IPs=("${LOCAL_HOST}")
fi

NGPU=${NGPU:-8}
MASTER_ADDR=${MASTER_ADDR:-${IPs[0]}}
MASTER_PORT=${MASTER_PORT:-6300}
NNODES=${NNODES:-${#IPs[@]}}
NODE_RANK=${NODE_RANK:-}
if [[ -z "${NODE_RANK}" ]]; then
    for i in "${!IPs[@]}"; do
        if [[ "${LOCAL_HOST}" == "${IPs[$i]}" ]]; then NODE_RANK=$i; break; fi
    done
fi
if [[ -z "${NODE_RANK}" ]]; then
    echo "[Error] this host (${LOCAL_HOST}) is not in NODE_IPS and NODE_RANK is not set" >&2
    exit 1
fi
echo "node ${NODE_RANK}/${NNODES} (${LOCAL_HOST}), master ${MASTER_ADDR}:${MASTER_PORT}"

MODULE=${MODULE:-deepseek_v32}
CONFIG=${CONFIG:-deepseek_v32_671b_61layers_4k}
TRAIN_FILE=${TRAIN_FILE:-titan_b200.entry}

cd "$(dirname "$0")/.."
mkdir -p logs
logfile="logs/${CONFIG}_$(date +%Y%m%d%H%M)_node${NODE_RANK}_${LOCAL_HOST//./_}.log"

python -m torch.distributed.run --nnodes="${NNODES}" --node-rank="${NODE_RANK}" --nproc-per-node="${NGPU}" \
    --master-addr="${MASTER_ADDR}" --master-port="${MASTER_PORT}" \
    --local-ranks-filter "${LOG_RANK}" --role rank --tee 3 \
    -m "${TRAIN_FILE}" --module "${MODULE}" --config "${CONFIG}" "$@" 2>&1 | tee -a "${logfile}"
