#!/usr/bin/env bash
# Smoke tier: the end-to-end feature matrix (tests/integration/run_matrix.py).  Every case trains a debug model for a
# few steps through the real launcher; the runner fails a case on a non-zero exit, a traceback, a NaN / Inf loss, too
# few logged steps or a timeout.  Without a GPU the host-only subset runs on gloo ranks.
#
#   .ci/smoke_test.sh                       all cases that fit this machine
#   .ci/smoke_test.sh --case llama3_tp      one case (arguments go to the runner)
set -euo pipefail

PROJECT_ROOT="$(cd "$(dirname "$0")/.." && pwd)"
REPORT_DIR="${REPORT_DIR:-${PROJECT_ROOT}/test_reports/integration}"
TIMEOUT_SECONDS="${TIMEOUT_SECONDS:-600}"
cd "$PROJECT_ROOT"

python -c "import __graft_entry__ as g; g.build()"
start=$(date +%s)
set +e
python tests/integration/run_matrix.py "$REPORT_DIR" --timeout "$TIMEOUT_SECONDS" "$@"
rc=$?
set -e
echo "smoke tier finished in $(( $(date +%s) - start ))s; report: $REPORT_DIR/report.json"
if [[ $rc -ne 0 ]]; then
    echo "--- failing cases ---"
    python - "$REPORT_DIR/report.json" <<'PY'
import json, sys
for c in json.load(open(sys.argv[1]))["cases"]:
    if c["status"] == "failed":
        print(f"{c['case']}: {c['reason']}")
PY
fi
exit $rc
