"""Read CUDA allocator snapshots written by the trainer (``--profiling.enable_memory_snapshot``: one
``rank<R>_memory_snapshot.pickle`` per rank under ``<dump_folder>/memory_snapshot/iteration_N/``) and say where the
memory went — the first tool to reach for after an out-of-memory error.

    python scripts/analyze_memory_snapshot.py SNAPSHOT.pickle                 # one snapshot
    python scripts/analyze_memory_snapshot.py BEFORE.pickle AFTER.pickle      # what changed between two
    python scripts/analyze_memory_snapshot.py S1.pickle S2.pickle S3.pickle   # three or more: steady growth = leak
    python scripts/analyze_memory_snapshot.py SNAPSHOT.pickle --json --top-n 20

For every snapshot the report gives
  * totals: reserved, allocated (live blocks), active (live + pending free), the free remainder inside reserved
    segments and the fragmentation ratio ``1 - allocated / reserved``;
  * a split of live bytes by what the allocating Python / C++ frames say the block is: parameters, gradients,
    optimizer state, activations (forward), backward temporaries, communication buffers, other;
  * the largest live blocks with the innermost frames that own them;
  * the peak of the recorded allocation timeline (``device_traces``): when it happened, what was allocated just
    before it, and whether the end of the trace sits well above its start (growth that survives a whole step);
  * fragmentation detail: free blocks inside segments, the largest of them, the share of small (< 1 MiB) free blocks.

The snapshot format is the dictionary of ``torch.cuda.memory._snapshot()``: ``segments`` (each with ``blocks`` of
``state`` / ``size`` / ``frames``) and ``device_traces`` (a list of alloc / free events per device).

(reference: .agents/skills/oom-analysis/scripts/analyze_snapshot.py — the same questions asked of NPU snapshots.)
"""

from __future__ import annotations

import argparse
import json
import pickle
import sys
from collections import defaultdict
from dataclasses import asdict, dataclass, field

MiB = 1 << 20
GiB = 1 << 30
SMALL_BLOCK = 1 * MiB

# (category, substrings looked for in "filename:function" of the frames, innermost first; first match wins)
CATEGORY_RULES: list[tuple[str, tuple[str, ...]]] = [
    ("optimizer", ("optim/", "optimizer", "adamw", "muon", "_init_group", "swap_optimizer", "exp_avg")),
    ("communication", ("distributed_c10d", "symm_mem", "fused_comm", "all_gather", "reduce_scatter", "all_to_all",
                       "nccl", "ProcessGroup", "fsdp_collectives", "_fsdp_collectives", "moe_comm")),
    ("gradient", ("accumulate_grad", "AccumulateGrad", "_fsdp_param_group.py:post_backward", "foreach_reduce",
                  "unsharded_grad", "clip_grad")),
    ("backward", ("autograd/function.py:apply", "autograd/graph.py", "_engine_run_backward", ":backward",
                  "Backward0", "Backward1")),
    ("parameter", ("init_weights", "reset_parameters", "_apply", "to_empty", "checkpoint/", "load_state_dict",
                   "fsdp_param.py", "_fsdp_param.py", "init_unsharded_param", "alloc_all_gather_outputs")),
    ("activation", ("forward", "__call__", "_call_impl", "checkpoint_wrapper", "models/")),
]
CATEGORIES = [c for c, _ in CATEGORY_RULES] + ["other"]


def load_snapshot(path: str) -> dict:
    with open(path, "rb") as f:
        snap = pickle.load(f)
    if not isinstance(snap, dict) or "segments" not in snap:
        raise ValueError(f"{path}: not an allocator snapshot (no 'segments' key)")
    return snap


def frame_label(fr: dict) -> str:
    return f"{fr.get('filename', '?')}:{fr.get('name', '?')}:{fr.get('line', 0)}"


def categorize(frames: list[dict] | None) -> str:
    """Name the kind of memory a block holds from the frames that allocated it."""
    if not frames:
        return "other"
    labels = [f"{fr.get('filename', '')}:{fr.get('name', '')}" for fr in frames]
    for cat, needles in CATEGORY_RULES:
        for lab in labels:
            if any(n in lab for n in needles):
                return cat
    return "other"


def own_frames(frames: list[dict] | None, depth: int = 4) -> list[str]:
    """The innermost frames outside torch's own plumbing: the lines a user can act on."""
    if not frames:
        return []
    skip = ("torch/nn/modules/module.py", "torch/autograd/", "torch/_ops.py", "torch/utils/_contextlib.py",
            "torch/_tensor.py", "torch/_compile.py", "<frozen", "??")
    keep = [frame_label(fr) for fr in frames if fr.get("filename") and not any(s in fr["filename"] for s in skip)]
    return (keep or [frame_label(fr) for fr in frames])[:depth]


@dataclass
class BlockInfo:
    size: int
    category: str
    frames: list[str]


@dataclass
class Fragmentation:
    free_bytes: int = 0
    free_blocks: int = 0
    largest_free: int = 0
    small_free_blocks: int = 0
    small_free_bytes: int = 0
    segments: int = 0
    segments_fully_free: int = 0


@dataclass
class Timeline:
    events: int = 0
    start_bytes: int = 0
    end_bytes: int = 0
    peak_bytes: int = 0
    peak_event: int = 0
    peak_share_of_trace: float = 0.0
    ooms: int = 0
    before_peak: list[dict] = field(default_factory=list)
    growth_bytes: int = 0


@dataclass
class Report:
    path: str
    device: int
    reserved: int
    allocated: int
    active: int
    fragmentation_ratio: float
    by_category: dict[str, int]
    top_blocks: list[BlockInfo]
    fragmentation: Fragmentation
    timeline: Timeline


def _block_frames(block: dict) -> list[dict] | None:
    if block.get("frames"):
        return block["frames"]
    hist = block.get("history")  # older snapshot layout: frames live in the newest history entry
    if hist:
        return hist[-1].get("frames")
    return None


def analyze_timeline(traces: list[dict], top_n: int) -> Timeline:
    tl = Timeline(events=len(traces))
    live = 0
    lowest = 0
    sizes: list[tuple[int, int, dict]] = []  # (event index, running bytes, event)
    for i, ev in enumerate(traces):
        action, size = ev.get("action", ""), int(ev.get("size", 0))
        if action == "alloc":
            live += size
        elif action in ("free_completed", "free"):  # "free_requested" precedes it and moves no bytes
            live -= size
        elif action == "oom":
            tl.ooms += 1
        lowest = min(lowest, live)
        sizes.append((i, live, ev))
        if live > tl.peak_bytes:
            tl.peak_bytes, tl.peak_event = live, i
    if not traces:
        return tl
    tl.start_bytes, tl.end_bytes = -lowest, live - lowest
    tl.peak_bytes -= lowest
    tl.peak_share_of_trace = (tl.peak_event + 1) / len(traces)
    tl.growth_bytes = tl.end_bytes - tl.start_bytes
    window = [ev for _, _, ev in sizes[max(0, tl.peak_event - 200): tl.peak_event + 1] if ev.get("action") == "alloc"]
    window.sort(key=lambda ev: -int(ev.get("size", 0)))
    for ev in window[:top_n]:
        tl.before_peak.append({"size": int(ev.get("size", 0)), "category": categorize(ev.get("frames")),
                               "frames": own_frames(ev.get("frames"))})
    return tl


def analyze(snap: dict, path: str = "", device: int | None = None, top_n: int = 10) -> Report:
    segs = snap.get("segments", [])
    if device is None:
        device = min((s.get("device", 0) for s in segs), default=0)
    segs = [s for s in segs if s.get("device", 0) == device]
    reserved = allocated = active = 0
    by_cat: dict[str, int] = defaultdict(int)
    blocks: list[BlockInfo] = []
    frag = Fragmentation(segments=len(segs))
    for seg in segs:
        reserved += int(seg.get("total_size", 0))
        seg_live = 0
        for b in seg.get("blocks", []):
            size, state = int(b.get("size", 0)), b.get("state", "")
            if state == "active_allocated":
                frames = _block_frames(b)
                cat = categorize(frames)
                allocated += size
                active += size
                seg_live += size
                by_cat[cat] += size
                blocks.append(BlockInfo(size, cat, own_frames(frames)))
            elif state == "active_pending_free":
                active += size
                seg_live += size
            else:  # inactive: free space inside a reserved segment
                frag.free_bytes += size
                frag.free_blocks += 1
                frag.largest_free = max(frag.largest_free, size)
                if size < SMALL_BLOCK:
                    frag.small_free_blocks += 1
                    frag.small_free_bytes += size
        if seg_live == 0:
            frag.segments_fully_free += 1
    blocks.sort(key=lambda b: -b.size)
    traces = snap.get("device_traces") or []
    trace = traces[device] if device < len(traces) else []
    return Report(path=path, device=device, reserved=reserved, allocated=allocated, active=active,
                  fragmentation_ratio=(1 - allocated / reserved) if reserved else 0.0,
                  by_category={c: by_cat.get(c, 0) for c in CATEGORIES}, top_blocks=blocks[:top_n],
                  fragmentation=frag, timeline=analyze_timeline(trace, top_n))


def fmt_bytes(n: float) -> str:
    sign = "-" if n < 0 else ""
    n = abs(n)
    if n >= GiB:
        return f"{sign}{n / GiB:.2f} GiB"
    if n >= MiB:
        return f"{sign}{n / MiB:.1f} MiB"
    return f"{sign}{n / 1024:.1f} KiB"


def render(r: Report) -> str:
    out = [f"== {r.path or 'snapshot'} (device {r.device}) ==",
           f"reserved {fmt_bytes(r.reserved)}   allocated {fmt_bytes(r.allocated)}   active {fmt_bytes(r.active)}   "
           f"free inside segments {fmt_bytes(r.fragmentation.free_bytes)}   fragmentation {100 * r.fragmentation_ratio:.1f}%",
           "", "live bytes by kind:"]
    for cat, n in sorted(r.by_category.items(), key=lambda kv: -kv[1]):
        share = 100 * n / r.allocated if r.allocated else 0.0
        out.append(f"  {cat:<14}{fmt_bytes(n):>12}  {share:5.1f}%")
    out += ["", f"largest live blocks (top {len(r.top_blocks)}):"]
    for i, b in enumerate(r.top_blocks, 1):
        out.append(f"  {i:>2}. {fmt_bytes(b.size):>10}  [{b.category}]")
        out += [f"        {fr}" for fr in b.frames]
    f = r.fragmentation
    out += ["", "fragmentation:",
            f"  {f.free_blocks} free blocks in {f.segments} segments ({f.segments_fully_free} segments entirely free); "
            f"largest free block {fmt_bytes(f.largest_free)}",
            f"  free blocks under 1 MiB: {f.small_free_blocks} ({fmt_bytes(f.small_free_bytes)})"]
    if f.free_bytes and f.largest_free < 0.25 * f.free_bytes:
        out.append("  -> free space is scattered: the largest hole is under a quarter of it; an allocation larger than "
                   "that hole fails although the bytes exist (try PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True)")
    t = r.timeline
    if t.events:
        out += ["", f"timeline ({t.events} events, {t.ooms} out-of-memory events):",
                f"  start {fmt_bytes(t.start_bytes)} -> peak {fmt_bytes(t.peak_bytes)} at {100 * t.peak_share_of_trace:.0f}% "
                f"of the trace -> end {fmt_bytes(t.end_bytes)}"]
        if t.growth_bytes > 0.05 * max(t.peak_bytes, 1):
            out.append(f"  -> the trace ends {fmt_bytes(t.growth_bytes)} above its start: memory that outlives the "
                       "recorded window (first steps allocate state; in later steps this is a leak)")
        if t.before_peak:
            out.append("  largest allocations in the 200 events before the peak:")
            for ev in t.before_peak:
                where = ev["frames"][0] if ev["frames"] else "?"
                out.append(f"    {fmt_bytes(ev['size']):>10}  [{ev['category']}]  {where}")
    return "\n".join(out)


def render_diff(a: Report, b: Report, label_a: str, label_b: str) -> str:
    out = [f"== {label_b} minus {label_a} =="]
    for name in ("reserved", "allocated", "active"):
        va, vb = getattr(a, name), getattr(b, name)
        out.append(f"  {name:<10}{fmt_bytes(va):>12} -> {fmt_bytes(vb):>12}   ({fmt_bytes(vb - va)})")
    out.append(f"  fragmentation {100 * a.fragmentation_ratio:.1f}% -> {100 * b.fragmentation_ratio:.1f}%")
    out.append("  by kind:")
    for cat in CATEGORIES:
        d = b.by_category[cat] - a.by_category[cat]
        if d:
            out.append(f"    {cat:<14}{fmt_bytes(d):>12}")
    return "\n".join(out)


def render_leak(reports: list[Report]) -> str:
    series = [r.allocated for r in reports]
    steps = [b - a for a, b in zip(series, series[1:])]
    out = ["== growth across snapshots ==", "  allocated: " + " -> ".join(fmt_bytes(v) for v in series)]
    if all(s > 0 for s in steps):
        out.append(f"  -> allocated memory grew in every interval (mean {fmt_bytes(sum(steps) / len(steps))} each): a leak")
        for cat in CATEGORIES:
            d = reports[-1].by_category[cat] - reports[0].by_category[cat]
            if d > 0:
                out.append(f"     {cat:<14}{fmt_bytes(d):>12}")
    else:
        out.append("  -> no monotonic growth")
    return "\n".join(out)


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("snapshots", nargs="+", help="1 = analyse, 2 = compare, 3+ = look for steady growth")
    ap.add_argument("--json", action="store_true", help="print the structured result instead of the text report")
    ap.add_argument("--top-n", type=int, default=10)
    ap.add_argument("--device", type=int, default=None, help="device index inside the snapshot (default: the first)")
    ap.add_argument("--label-a", default="baseline")
    ap.add_argument("--label-b", default="modified")
    args = ap.parse_args(argv)
    reports = [analyze(load_snapshot(p), p, args.device, args.top_n) for p in args.snapshots]
    if args.json:
        print(json.dumps([asdict(r) for r in reports], indent=1))
        return 0
    for r in reports:
        print(render(r))
        print()
    if len(reports) == 2:
        print(render_diff(reports[0], reports[1], args.label_a, args.label_b))
    elif len(reports) > 2:
        print(render_leak(reports))
    return 0


if __name__ == "__main__":
    sys.exit(main())
