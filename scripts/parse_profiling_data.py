"""Summarise profiler traces written by the trainer (``<dump_folder>/profile_traces/iteration_N/*.json[.gz]``).

    python scripts/parse_profiling_data.py outputs/profile_traces/iteration_7 [--top 30]

Prints, per trace file, total device time and the kernels with the largest summed duration (count, total ms, share),
split into this framework's kernels (names with ``tb_`` / ``gemm_tcgen05`` / ``_kernel<`` from the in-tree library) and
library kernels — the first place to look when a step is slower than expected.

(reference: scripts/parse_profiling_data.py — offline parsing of traces collected with online parsing disabled)
"""

from __future__ import annotations

import argparse
import collections
import glob
import gzip
import json
import os

OURS = ("gemm_tcgen05", "rmsnorm", "rope_", "swiglu", "cross_entropy", "adamw_multi", "topk_select", "moe_", "mhc_",
        "router_topk", "rs_reduce", "castscale", "bwd_cta_kernel", "bwd_warp_kernel", "fwd_rowreg")


def load_events(path: str):
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rt") as f:
        data = json.load(f)
    return data["traceEvents"] if isinstance(data, dict) else data


def summarise(path: str, top: int) -> None:
    by_name: dict[str, list[float]] = collections.defaultdict(lambda: [0, 0.0])
    for ev in load_events(path):
        if ev.get("ph") == "X" and ev.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset"):
            rec = by_name[ev.get("name", "?")]
            rec[0] += 1
            rec[1] += float(ev.get("dur", 0.0)) / 1000.0
    total = sum(v[1] for v in by_name.values())
    ours = sum(v[1] for k, v in by_name.items() if any(t in k for t in OURS))
    print(f"== {path}: {len(by_name)} kernels, {total:.2f} ms on device, {ours:.2f} ms ({100 * ours / max(total, 1e-9):.1f} %) "
          "in in-tree kernels")
    print(f"{'ms':>10} {'share':>7} {'count':>7}  name")
    for name, (cnt, ms) in sorted(by_name.items(), key=lambda kv: -kv[1][1])[:top]:
        mark = "*" if any(t in name for t in OURS) else " "
        print(f"{ms:10.3f} {100 * ms / max(total, 1e-9):6.1f}% {cnt:7d} {mark}{name[:110]}")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("path", help="a trace file or a folder of traces")
    ap.add_argument("--top", type=int, default=30)
    a = ap.parse_args()
    files = [a.path] if os.path.isfile(a.path) else sorted(
        glob.glob(os.path.join(a.path, "**", "*.json"), recursive=True) +
        glob.glob(os.path.join(a.path, "**", "*.json.gz"), recursive=True))
    if not files:
        raise SystemExit(f"no trace files under {a.path!r}")
    for f in files:
        summarise(f, a.top)
