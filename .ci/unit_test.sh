#!/usr/bin/env bash
# Unit tier: cross-compile the CUDA library for sm_100a (needs nvcc, no GPU), then the tests that need no device.
# On a machine with a B200 the kernel numerics tests (`-m gpu`) run as well.
#
#   .ci/unit_test.sh              CPU tier (+ GPU tier when a device is visible)
#   TIER=cpu .ci/unit_test.sh     CPU tier only
#   REPORT_DIR=out .ci/unit_test.sh
set -euo pipefail

PROJECT_ROOT="$(cd "$(dirname "$0")/.." && pwd)"
REPORT_DIR="${REPORT_DIR:-${PROJECT_ROOT}/test_reports}"
TIER="${TIER:-auto}"
TIMEOUT_SECONDS="${TIMEOUT_SECONDS:-3600}"
cd "$PROJECT_ROOT"
mkdir -p "$REPORT_DIR"

echo "== build (sm_100a) =="
python -c "import __graft_entry__ as g; g.build()"

echo "== unit tests without a device =="
timeout "$TIMEOUT_SECONDS" python -m pytest tests -q -m "not gpu" --junitxml "$REPORT_DIR/unit_cpu.xml"

has_gpu=$(python -c "import torch; print(int(torch.cuda.is_available()))")
if [[ "$TIER" != "cpu" && "$has_gpu" == "1" ]]; then
    echo "== kernel and multi-GPU tests =="
    timeout "$TIMEOUT_SECONDS" python -m pytest tests -q -m gpu --junitxml "$REPORT_DIR/unit_gpu.xml"
else
    echo "no GPU visible (or TIER=cpu): the -m gpu tier was skipped"
fi
