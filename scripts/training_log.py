"""Work with the trainer's step lines

    step: 10  loss:  7.9312  grad_norm:  1.2043  memory: 41.07GiB(22.94%)  tps: 19,978  tflops: 917.21  mfu: 40.77%  elapsed_time_per_step: 0.4101s

Three sub-commands:

    python scripts/training_log.py summary RUN.log [--skip 5]
        steps seen, last loss, mean / best tokens-per-second, MFU and step time after the first ``--skip`` logged
        steps, peak memory.

    python scripts/training_log.py compare --baseline A.log --candidate B.log [--tolerance 1e-5]
                                           [--metrics loss grad_norm] [--output DIR]
        step-by-step absolute and relative differences of the chosen metrics over the steps both logs have; writes
        ``compare_report.md`` and ``compare_report.json`` into DIR and exits 1 when any difference exceeds the
        tolerance — the check to run before merging a change that must not move the numerics (same seed, deterministic
        mode, same parallel layout).

    python scripts/training_log.py plot --log-a A.log [--log-b B.log] [--metrics loss grad_norm tps] [--output OUT.svg]
                                        [--smooth 0.0] [--title TEXT]
        one panel per metric as a standalone SVG (no plotting library needed); with two logs both curves share each
        panel and a further panel shows their difference.

(reference: .agents/skills/premerge-accuracy-check/scripts/{loss_compare,generate_report}.py and
.agents/skills/training-log-visualization/scripts/{plot_training_logs,train_log_plot}.py)
"""

from __future__ import annotations

import argparse
import json
import math
import os
import re
import sys

STEP_RE = re.compile(r"step:\s*(\d+)\s")
FIELD_RES = {
    "loss": re.compile(r"\bloss:\s*([-+0-9.eE]+|nan|inf)"),
    "grad_norm": re.compile(r"\bgrad_norm:\s*([-+0-9.eE]+|nan|inf)"),
    "memory_gib": re.compile(r"\bmemory:\s*([0-9.]+)GiB"),
    "memory_pct": re.compile(r"\bmemory:\s*[0-9.]+GiB\(([0-9.]+)%\)"),
    "tps": re.compile(r"\btps:\s*([0-9,]+)"),
    "tflops": re.compile(r"\btflops:\s*([0-9.]+)"),
    "mfu": re.compile(r"\bmfu:\s*([0-9.]+)%"),
    "step_time": re.compile(r"\belapsed_time_per_step:\s*([0-9.]+)s"),
}
ANSI_RE = re.compile(r"\x1b\[[0-9;]*m")
DEFAULT_COMPARE = ["loss", "grad_norm"]
DEFAULT_TOLERANCE = 1e-5


def parse_log(path: str) -> dict[int, dict[str, float]]:
    """step → {metric: value}; a step logged twice (restart from a checkpoint) keeps its LAST line."""
    records: dict[int, dict[str, float]] = {}
    with open(path, errors="replace") as f:
        for line in f:
            line = ANSI_RE.sub("", line)
            m = STEP_RE.search(line)
            if not m or "loss:" not in line:
                continue
            rec: dict[str, float] = {}
            for key, rx in FIELD_RES.items():
                fm = rx.search(line)
                if fm:
                    rec[key] = float(fm.group(1).replace(",", ""))
            records[int(m.group(1))] = rec
    return records


def series(records: dict[int, dict[str, float]], metric: str) -> tuple[list[int], list[float]]:
    steps = [s for s in sorted(records) if metric in records[s]]
    return steps, [records[s][metric] for s in steps]


# ------------------------------------------------------------------ summary

def summarize(records: dict[int, dict[str, float]], skip: int = 5) -> dict:
    steps = sorted(records)
    if not steps:
        return {"steps_logged": 0}
    steady = steps[skip:] or steps[-1:]
    out = {"steps_logged": len(steps), "first_step": steps[0], "last_step": steps[-1],
           "last_loss": records[steps[-1]].get("loss"), "skipped": min(skip, len(steps) - 1)}
    for key in ("tps", "tflops", "mfu", "step_time"):
        vals = [records[s][key] for s in steady if key in records[s]]
        if vals:
            out[f"{key}_mean"] = sum(vals) / len(vals)
            out[f"{key}_best"] = min(vals) if key == "step_time" else max(vals)
    mem = [records[s]["memory_gib"] for s in steps if "memory_gib" in records[s]]
    if mem:
        out["memory_gib_peak"] = max(mem)
    bad = [s for s in steps if not math.isfinite(records[s].get("loss", 0.0))]
    if bad:
        out["non_finite_loss_steps"] = bad
    return out


# ------------------------------------------------------------------ compare

def compare(base: dict[int, dict[str, float]], cand: dict[int, dict[str, float]], metrics: list[str],
            tolerance: float) -> dict:
    common = sorted(set(base) & set(cand))
    result = {"tolerance": tolerance, "steps_compared": len(common), "only_in_baseline": sorted(set(base) - set(cand)),
              "only_in_candidate": sorted(set(cand) - set(base)), "metrics": {}, "passed": bool(common)}
    for metric in metrics:
        rows = []
        worst_abs = worst_rel = 0.0
        first_bad = None
        for s in common:
            if metric not in base[s] or metric not in cand[s]:
                continue
            a, b = base[s][metric], cand[s][metric]
            if math.isnan(a) and math.isnan(b):
                d = rel = 0.0
            else:
                d = abs(a - b)
                rel = d / max(abs(a), 1e-12)
            if not d <= tolerance and first_bad is None:  # `not <=` also catches NaN on one side
                first_bad = s
            if not math.isnan(d):
                worst_abs, worst_rel = max(worst_abs, d), max(worst_rel, rel)
            rows.append({"step": s, "baseline": a, "candidate": b, "abs_diff": d, "rel_diff": rel})
        ok = first_bad is None and bool(rows)
        result["metrics"][metric] = {"passed": ok, "max_abs_diff": worst_abs, "max_rel_diff": worst_rel,
                                     "first_step_over_tolerance": first_bad, "rows": rows}
        result["passed"] = result["passed"] and ok
    return result


def compare_markdown(res: dict, base_path: str, cand_path: str, max_rows: int = 40) -> str:
    out = ["# Training-log comparison", "", f"* baseline: `{base_path}`", f"* candidate: `{cand_path}`",
           f"* steps compared: {res['steps_compared']}   tolerance: {res['tolerance']:g}",
           f"* result: **{'PASS' if res['passed'] else 'FAIL'}**", ""]
    if res["only_in_baseline"] or res["only_in_candidate"]:
        out += [f"Steps only in the baseline: {res['only_in_baseline'][:20]}; only in the candidate: "
                f"{res['only_in_candidate'][:20]}", ""]
    for metric, m in res["metrics"].items():
        out += [f"## {metric}: {'pass' if m['passed'] else 'FAIL'}", "",
                f"max |diff| {m['max_abs_diff']:.3e}, max relative {m['max_rel_diff']:.3e}"
                + (f", first step over tolerance: {m['first_step_over_tolerance']}"
                   if m["first_step_over_tolerance"] is not None else ""), "",
                "| step | baseline | candidate | abs diff | rel diff |", "|---|---|---|---|---|"]
        rows = m["rows"]
        if len(rows) > max_rows:  # keep the head, the tail and every row over the tolerance
            keep = {r["step"] for r in rows[: max_rows // 2]} | {r["step"] for r in rows[-max_rows // 2:]}
            rows = [r for r in rows if r["step"] in keep or not r["abs_diff"] <= res["tolerance"]]
        for r in rows:
            out.append(f"| {r['step']} | {r['baseline']:.6f} | {r['candidate']:.6f} | {r['abs_diff']:.3e} | "
                       f"{r['rel_diff']:.3e} |")
        out.append("")
    return "\n".join(out)


# ------------------------------------------------------------------ plot (plain SVG)

PALETTE = ("#1f77b4", "#d62728", "#2ca02c")


def ema(values: list[float], alpha: float) -> list[float]:
    if not values or alpha <= 0:
        return list(values)
    out, acc = [], values[0]
    for v in values:
        acc = alpha * acc + (1 - alpha) * v
        out.append(acc)
    return out


def _ticks(lo: float, hi: float, n: int = 5) -> list[float]:
    if not math.isfinite(lo) or not math.isfinite(hi) or hi <= lo:
        return [lo]
    raw = (hi - lo) / n
    mag = 10 ** math.floor(math.log10(raw))
    step = min((m * mag for m in (1, 2, 5, 10) if m * mag >= raw), default=raw)
    first = math.ceil(lo / step) * step
    return [first + i * step for i in range(int((hi - first) / step) + 1)]


def _panel(x0: int, y0: int, w: int, h: int, title: str, curves: list[tuple[str, list[int], list[float], str]]) -> str:
    pts = [(s, v) for _, ss, vs, _ in curves for s, v in zip(ss, vs) if math.isfinite(v)]
    if not pts:
        return f'<text x="{x0}" y="{y0 + 20}" font-size="12">{title}: no data</text>'
    xs, ys = [p[0] for p in pts], [p[1] for p in pts]
    xlo, xhi, ylo, yhi = min(xs), max(xs), min(ys), max(ys)
    if xhi == xlo:
        xhi = xlo + 1
    if yhi == ylo:
        ylo, yhi = ylo - 0.5, yhi + 0.5
    pad = 0.05 * (yhi - ylo)
    ylo, yhi = ylo - pad, yhi + pad
    px = lambda s: x0 + (s - xlo) / (xhi - xlo) * w  # noqa: E731
    py = lambda v: y0 + h - (v - ylo) / (yhi - ylo) * h  # noqa: E731
    out = [f'<rect x="{x0}" y="{y0}" width="{w}" height="{h}" fill="none" stroke="#888"/>',
           f'<text x="{x0}" y="{y0 - 6}" font-size="13" font-weight="bold">{title}</text>']
    for t in _ticks(ylo, yhi):
        out.append(f'<line x1="{x0}" x2="{x0 + w}" y1="{py(t):.1f}" y2="{py(t):.1f}" stroke="#ddd"/>')
        out.append(f'<text x="{x0 - 4}" y="{py(t) + 4:.1f}" font-size="10" text-anchor="end">{t:.4g}</text>')
    for t in _ticks(xlo, xhi):
        out.append(f'<text x="{px(t):.1f}" y="{y0 + h + 12}" font-size="10" text-anchor="middle">{t:.0f}</text>')
    for i, (label, ss, vs, color) in enumerate(curves):
        path = " ".join(f"{px(s):.1f},{py(v):.1f}" for s, v in zip(ss, vs) if math.isfinite(v))
        out.append(f'<polyline fill="none" stroke="{color}" stroke-width="1.4" points="{path}"/>')
        out.append(f'<text x="{x0 + w - 4}" y="{y0 + 14 + 13 * i}" font-size="11" text-anchor="end" fill="{color}">'
                   f'{label}</text>')
    return "\n".join(out)


def plot_svg(logs: list[tuple[str, dict[int, dict[str, float]]]], metrics: list[str], smooth: float = 0.0,
             title: str | None = None) -> str:
    panels = []
    for metric in metrics:
        curves = []
        for i, (label, rec) in enumerate(logs):
            ss, vs = series(rec, metric)
            curves.append((label, ss, ema(vs, smooth), PALETTE[i % len(PALETTE)]))
        panels.append((metric, curves))
        if len(logs) == 2:
            (_, a), (_, b) = logs
            common = [s for s in sorted(set(a) & set(b)) if metric in a[s] and metric in b[s]]
            if common:
                panels.append((f"{metric}: {logs[1][0]} - {logs[0][0]}",
                               [("difference", common, [b[s][metric] - a[s][metric] for s in common], PALETTE[2])]))
    W, H, left, top, gap = 720, 200, 70, 50, 50
    height = top + len(panels) * (H + gap)
    body = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W + left + 30}" height="{height}" font-family="sans-serif">',
            '<rect width="100%" height="100%" fill="white"/>']
    if title:
        body.append(f'<text x="{left}" y="22" font-size="16" font-weight="bold">{title}</text>')
    for i, (name, curves) in enumerate(panels):
        body.append(_panel(left, top + i * (H + gap), W, H, name, curves))
    body.append("</svg>")
    return "\n".join(body)


# ------------------------------------------------------------------ CLI

def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    sp = sub.add_parser("summary")
    sp.add_argument("log")
    sp.add_argument("--skip", type=int, default=5, help="logged steps to leave out of the throughput averages")
    cp = sub.add_parser("compare")
    cp.add_argument("--baseline", required=True)
    cp.add_argument("--candidate", required=True)
    cp.add_argument("--output", default=os.getcwd())
    cp.add_argument("--tolerance", type=float, default=DEFAULT_TOLERANCE)
    cp.add_argument("--metrics", nargs="*", default=DEFAULT_COMPARE)
    pp = sub.add_parser("plot")
    pp.add_argument("--log-a", required=True)
    pp.add_argument("--log-b", default=None)
    pp.add_argument("--metrics", nargs="*", default=["loss", "grad_norm", "tps"])
    pp.add_argument("--output", default=None)
    pp.add_argument("--smooth", type=float, default=0.0, help="exponential smoothing factor in [0, 1)")
    pp.add_argument("--title", default=None)
    args = ap.parse_args(argv)

    if args.cmd == "summary":
        print(json.dumps(summarize(parse_log(args.log), args.skip), indent=1))
        return 0
    if args.cmd == "compare":
        for label, path in (("baseline", args.baseline), ("candidate", args.candidate)):
            if not os.path.isfile(path):
                print(f"{label} log not found: {path}", file=sys.stderr)
                return 2
        res = compare(parse_log(args.baseline), parse_log(args.candidate), args.metrics, args.tolerance)
        os.makedirs(args.output, exist_ok=True)
        with open(os.path.join(args.output, "compare_report.json"), "w") as f:
            json.dump(res, f, indent=1)
        with open(os.path.join(args.output, "compare_report.md"), "w") as f:
            f.write(compare_markdown(res, args.baseline, args.candidate))
        for metric, m in res["metrics"].items():
            print(f"{metric}: {'pass' if m['passed'] else 'FAIL'}  max|diff| {m['max_abs_diff']:.3e}  "
                  f"max rel {m['max_rel_diff']:.3e}")
        print("PASS" if res["passed"] else "FAIL")
        return 0 if res["passed"] else 1
    logs = [(os.path.basename(args.log_a), parse_log(args.log_a))]
    if args.log_b:
        logs.append((os.path.basename(args.log_b), parse_log(args.log_b)))
    out = args.output or os.path.splitext(args.log_a)[0] + ".svg"
    with open(out, "w") as f:
        f.write(plot_svg(logs, args.metrics, args.smooth, args.title))
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
