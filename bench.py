"""Headline benchmark: Llama-3 8B pretraining step (FSDP2 over the N GPUs, bf16 params/compute, fp32 gradient
reduction, seq 8192, local batch 1, selective activation checkpointing, AdamW) — whole-job training tokens/s,
device-timed.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run)
    python bench.py --impl reference ...                      (the unmodified reference, if it can run here)
    python bench.py --impl baseline ...                       (this framework on library ops only)

One invocation measures up to three arms back to back in the same process(es), each on a freshly built trainer:
  1. the product arm (`value`, `e2e`): recipe `llama3_8b` (this framework's kernels, selective checkpointing);
  2. the library arm (`baseline`): the same model, checkpointing rule, reshard policy and optimizer maths on
     cuBLAS / cuDNN-SDPA / torch fused AdamW / NCCL only; `vs_baseline` = product tokens/s ÷ library tokens/s;
  3. the product recipe without recomputation (`variants.activation_checkpoint_none`), reported beside the headline,
     never as `value`.
`--arms product` runs the first arm only.

Two timed regions of K steps each, both bracketed by barrier + synchronize and timed with CUDA
events, max over ranks:
  * `value`  – optimizer steps fed from batches already resident on the device;
  * `e2e`    – the same steps through `Trainer.train_step` with the real loader: every step copies
               its inputs from pinned host memory to the device and reads the loss back to the host.
Weights (16 GB) and activations are far larger than the 126 MB L2, so no explicit L2 flush is needed.
SM clocks and throttle reasons are sampled with nvidia-smi during the timed regions.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "train_tokens_per_sec"



def _compute_dtype(cfg) -> str:
    """The dtype the GEMMs run in: a recipe with a low-precision converter is reported as such, never as bf16."""
    names = [getattr(c, "name", str(c)) for c in cfg.model_converters.converters]
    base = "bf16" if cfg.training.dtype == "bfloat16" else cfg.training.dtype
    if "mxfp8" in names:
        return f"mxfp8 (block-scaled e4m3 GEMMs, fp32 accumulate; everything else {base})"
    if "quantize" in names:
        return f"quantised weights ({base} compute)"
    return base

def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "baseline", "reference"])
    ap.add_argument("--module", default="llama3")
    ap.add_argument("--config", default=None, help="recipe function; default llama3_8b (ours) / llama3_8b_baseline")
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--local-batch", type=int, default=None)
    ap.add_argument("--flavor", default=None, help="override the model flavor (smoke runs only)")
    ap.add_argument("--converters", default=None, help="comma-separated converter names overriding the recipe")
    ap.add_argument("--ac", default=None, choices=["none", "selective", "full"])
    ap.add_argument("--breakdown", type=int, default=0, metavar="ROWS",
                    help="after timing, profile one more step and write the top ROWS kernels by device time")
    ap.add_argument("--breakdown-out", default="kernel_breakdown.txt")
    ap.add_argument("--arms", default="product,library,noac",
                    help="which arms to measure in this invocation: product[,library][,noac]")
    ap.add_argument("--set", action="append", default=[], metavar="SECTION.FIELD=VALUE",
                    help="extra recipe overrides, e.g. --set parallelism.expert_parallel_degree=2 (repeatable)")
    return ap.parse_args()


# ----------------------------------------------------------------------------- reference arm
def reference_arm(args) -> int:
    """Run the unmodified reference from baseline/_ref through its own entry point, if importable."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    reason = None
    if not os.path.isdir(os.path.join(ref_dir, "torchtitan_npu")):
        reason = "baseline/_ref is absent (offline pip install of the reference was not done on this box)"
    else:
        sys.path.insert(0, ref_dir)
        try:
            import torchtitan_npu  # noqa: F401
        except BaseException as e:  # the reference hard-imports torch_npu / a newer torchtitan
            reason = f"reference cannot be imported here: {type(e).__name__}: {str(e).splitlines()[0][:160]}"
    if reason is None:
        reason = "reference imported but targets Ascend NPUs (torch_npu device ops); no CUDA path to run"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason}), flush=True)
    return 0


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.NamedTemporaryFile(prefix="clocks_", suffix=".csv", delete=False).name
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 8:
                        continue
                    try:
                        sm.append(float(parts[0]))
                        mx.append(float(parts[1]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                          "sw_power_cap"), parts[4:8]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            # under load = upper half of the samples (idle samples before/after the region drop out)
            loaded = sorted(sm)[len(sm) // 2:]
            out.update(sm_mhz=statistics.median(loaded), sm_max_mhz=max(mx), reasons=sorted(reasons),
                       samples=len(sm))
        return out


# ----------------------------------------------------------------------------- our arms
def build_config(args, impl: str, ac_override: str | None = None):
    from titan_b200.config.manager import resolve_recipe
    from titan_b200.protocols.converter import get_model_converter_config

    recipe = args.config if (args.config and impl == args.impl) else (
        "llama3_8b" if impl == "ours" else "llama3_8b_baseline")
    cfg = resolve_recipe(args.module, recipe)
    if args.seq_len:
        cfg.training.seq_len = args.seq_len
    if args.local_batch:
        cfg.training.local_batch_size = args.local_batch
    if args.flavor:
        cfg.model.flavor = args.flavor
    if args.converters is not None and impl == "ours":
        cfg.model_converters.converters = [get_model_converter_config(n) for n in args.converters.split(",") if n]
    if ac_override or args.ac:
        cfg.activation_checkpoint.mode = ac_override or args.ac
    if args.set:
        from titan_b200.config.manager import apply_overrides

        cfg = apply_overrides(cfg, [f"--{kv}" for kv in args.set])
    cfg.training.steps = 10 ** 9  # the bench drives steps itself; keeps the LR schedule in warm-up
    cfg.metrics.log_freq = 10 ** 9
    cfg.checkpoint.enable = False
    cfg.training.gc_freq = 10 ** 9
    return cfg, recipe


def run_arm(args, impl: str, *, ac_override: str | None = None, with_e2e: bool = True, sample_clocks: bool = True,
            breakdown: bool = False) -> dict:
    """Build a trainer for one arm, time it, tear it down.  Returns the measurements (identical on every rank)."""
    import gc

    import torch
    import torch.distributed as dist

    from titan_b200.ops import _lib

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg, recipe = build_config(args, impl, ac_override)
    torch.cuda.reset_peak_memory_stats()
    trainer = cfg.build()
    device = trainer.device
    K, W = args.steps, args.warmup

    def barrier():
        if dist.is_initialized():
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if not dist.is_initialized():
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    barrier()  # creates the communicator now: after warm-up the caching allocator may hold all free memory
    tokens_per_step_rank = cfg.training.local_batch_size * cfg.training.seq_len
    dp = trainer.dp_degree
    tokens_per_step = tokens_per_step_rank * dp

    # ---- region 1: device-resident inputs (kernel-side number)
    loader_iter = trainer.batch_generator(trainer.dataloader)
    staged = [next(loader_iter) for _ in range(2)]
    torch.cuda.synchronize()

    def staged_iter():
        i = 0
        while True:
            yield staged[i % len(staged)]
            i += 1

    sit = staged_iter()
    for _ in range(W):
        trainer.step += 1
        trainer.train_step(sit)
    barrier()
    sampler = ClockSampler(local_rank) if (rank == 0 and sample_clocks) else None
    launches0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        trainer.step += 1
        trainer.train_step(sit)
    e1.record()
    torch.cuda.synchronize()
    launches = _lib.launch_count() - launches0
    barrier()
    dev_ms = max_over_ranks(e0.elapsed_time(e1))

    # ---- region 2: end to end through the public loop: pinned host → device each step, loss → host each step
    e2e = None
    if with_e2e:
        losses = []
        barrier()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record()
        for _ in range(K):
            trainer.step += 1
            trainer.train_step(loader_iter)  # pulls a fresh pinned batch and copies it to the device
            loss_host = trainer._last_loss.to("cpu", non_blocking=False)
            losses.append(float(loss_host))
        e3.record()
        torch.cuda.synchronize()
        barrier()
        e2e_ms = max_over_ranks(e2.elapsed_time(e3))
        e2e = {"value": tokens_per_step / (e2e_ms / K / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": 2 * tokens_per_step_rank * 8,  # int64 inputs + labels per rank and step
               "d2h_bytes_per_step": 4 if cfg.training.dtype == "float32" else trainer._last_loss.element_size(),
               "ms_per_step": e2e_ms / K, "last_loss": losses[-1] if losses else None}
    clocks = sampler.stop() if sampler is not None else None

    if breakdown and args.breakdown:
        # one extra step under the profiler, after (never inside) the timed regions: shares of device time per kernel
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            trainer.step += 1
            trainer.train_step(sit)
            torch.cuda.synchronize()
        if rank == 0:
            table = prof.key_averages().table(sort_by="cuda_time_total", row_limit=args.breakdown,
                                              max_name_column_width=90)
            with open(args.breakdown_out, "w") as f:
                f.write(table)
            print(f"kernel breakdown of one step written to {args.breakdown_out}", file=sys.stderr)

    _lib.shared_status().raise_if_set("bench")  # any kernel-reported failure invalidates the run
    from titan_b200.utils.device import get_peak_flops

    ms_per_step = dev_ms / K
    value = tokens_per_step / (ms_per_step / 1e3)
    pd = trainer.parallel_dims
    par = "+".join(f"{n}{v}" for n, v in (("fsdp", pd.dp_shard), ("hsdp", pd.dp_replicate), ("tp", pd.tp),
                                           ("cp", pd.cp), ("pp", pd.pp), ("ep", pd.ep)) if v > 1) or "single"
    ac = cfg.activation_checkpoint
    out = {
        "impl": impl, "recipe": recipe, "value": value, "ms_per_step": ms_per_step, "e2e": e2e, "clocks": clocks,
        "gpu_launches": launches, "dtype": _compute_dtype(cfg),
        "mfu_pct_of_nominal_bf16": 100.0 * trainer.flops_per_token * (value / args.gpus) / get_peak_flops(),
        "max_memory_allocated_gib": torch.cuda.max_memory_allocated() / 2 ** 30,
        "config": {
            "model": f"{cfg.model.name}-{cfg.model.flavor}", "recipe": recipe,
            "global_batch": cfg.training.local_batch_size * dp, "seq_len": cfg.training.seq_len, "parallelism": par,
            "activation_checkpoint": ac.mode if ac.mode != "selective" else f"selective/{ac.selective_ac_option}",
            "fsdp_reshard_after_forward": cfg.parallelism.fsdp_reshard_after_forward,
            "fsdp_fused_collectives": bool(getattr(cfg.parallelism, "fsdp_fused_collectives", False)) and dp > 1,
            "optimizer": f"{cfg.optimizer.name}/{cfg.optimizer.implementation}",
            "converters": [getattr(c, "name", str(c)) for c in cfg.model_converters.converters],
            "l2": "inputs larger than L2 (weights + activations >> 126 MB); no explicit flush",
            "params": trainer.nparams,
        },
    }
    trainer.close()
    del trainer, staged, sit, loader_iter
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return out


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        print(json.dumps({"metric": METRIC, "error": "no CUDA device"}))
        return 1
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"--gpus {args.gpus} needs torch.distributed.run with --nproc-per-node {args.gpus}", file=sys.stderr)
            return 2
    rank = int(os.environ.get("RANK", "0"))
    os.environ.setdefault("LOG_RANK", "0")
    if args.warmup < 3:
        print("warning: fewer than 3 warm-up steps", file=sys.stderr)

    arms = set(args.arms.split(","))
    main_arm = run_arm(args, args.impl, breakdown=True)
    baseline = variant = None
    if args.impl == "ours" and "library" in arms:
        baseline = run_arm(args, "baseline", sample_clocks=False)
    if args.impl == "ours" and "noac" in arms and main_arm["config"]["activation_checkpoint"] != "none":
        variant = run_arm(args, "ours", ac_override="none", with_e2e=False, sample_clocks=False)

    if rank == 0:
        out = {
            "metric": METRIC, "value": main_arm["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_arm["ms_per_step"],
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (main_arm["value"] / baseline["value"]) if baseline else None,
            "dtype": main_arm["dtype"], "data": "synthetic", "impl": args.impl, "config": main_arm["config"],
            "tokens_per_sec_per_gpu": main_arm["value"] / args.gpus,
            "mfu_pct_of_nominal_bf16": main_arm["mfu_pct_of_nominal_bf16"],
            "max_memory_allocated_gib": main_arm["max_memory_allocated_gib"],
            "clocks": main_arm["clocks"], "e2e": main_arm["e2e"], "gpu_launches": main_arm["gpu_launches"],
        }
        if baseline:
            out["baseline"] = {
                "what": "same model, checkpointing rule, reshard policy and step on library kernels only (cuBLAS, "
                        "cuDNN SDPA, torch fused AdamW, NCCL), measured in this invocation after the product arm",
                "recipe": baseline["recipe"], "value": baseline["value"], "ms_per_step": baseline["ms_per_step"],
                "e2e_value": baseline["e2e"]["value"] if baseline["e2e"] else None,
                "e2e_vs_baseline": (main_arm["e2e"]["value"] / baseline["e2e"]["value"])
                if (baseline["e2e"] and main_arm["e2e"]) else None,
                "config": baseline["config"],
            }
        if variant:
            out["variants"] = {"activation_checkpoint_none": {
                "value": variant["value"], "ms_per_step": variant["ms_per_step"],
                "max_memory_allocated_gib": variant["max_memory_allocated_gib"],
                "note": "the product recipe without recomputation (fits in 180 GB); not the headline configuration"}}
        print(json.dumps(out), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
