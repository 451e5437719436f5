#!/usr/bin/env bash
# The same debug run with the Muon optimizer on the 2-D weight matrices (Newton-Schulz orthogonalised momentum;
# embeddings, norms, routers and 1-D parameters stay on AdamW).
set -euo pipefail
cd "$(dirname "$0")/../.."
NGPU=${NGPU:-8} MODULE=deepseek_v4 CONFIG=debug_deepseek_v4_single_node_1b ./scripts/run_train.sh \
    --optimizer.name Muon --optimizer.muon_momentum 0.95 --optimizer.muon_ns_steps 5 \
    --optimizer.muon_adjust_lr_fn match_rms_adamw "$@"
