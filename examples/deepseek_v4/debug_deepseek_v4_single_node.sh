#!/usr/bin/env bash
# Two steps of the 1B-class DeepSeek-V4 (`mini_1b`: hyper-connections, compressor + lightning-indexer attention, hash
# and score-routed experts, one MTP module) on one node: the quickest end-to-end check of every V4 component.
set -euo pipefail
cd "$(dirname "$0")/../.."
NGPU=${NGPU:-8} MODULE=deepseek_v4 CONFIG=debug_deepseek_v4_single_node_1b ./scripts/run_train.sh "$@"
