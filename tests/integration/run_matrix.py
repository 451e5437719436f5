"""End-to-end feature matrix: every case starts the real trainer for a few steps (one process per rank through
``torch.distributed.run``) and the runner reads the LOG, not just the exit code: a traceback, a NaN / Inf loss, fewer
logged steps than asked, or a timeout fails the case.  A JSON report and one log per case go to the output folder.

    python tests/integration/run_matrix.py out/                     every case that fits the visible devices
    python tests/integration/run_matrix.py out/ --case llama3_fsdp  one case
    python tests/integration/run_matrix.py out/ --device cpu        gloo ranks on the host (no GPU needed)
    python tests/integration/run_matrix.py out/ --list

Cases whose ``ranks`` exceed the visible GPUs are reported as skipped.  On ``--device cpu`` only cases marked
``cpu_ok`` run (the fused-kernel converters need a B200).

Plays the role of the reference's smoke-test integration runner (tests/smoke_tests/integration_test.py:40-260: a table
of override sets per model family × parallelism, launched through torchrun, with the log scanned afterwards by
.ci/smoke_test.sh:178-222).
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import os
import re
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


@dataclasses.dataclass(frozen=True)
class Case:
    name: str
    module: str
    config: str
    overrides: tuple[str, ...] = ()
    ranks: int = 2
    steps: int = 3
    cpu_ok: bool = False
    env: tuple[tuple[str, str], ...] = ()
    note: str = ""


def _c(*a, **k) -> Case:
    return Case(*a, **k)


CASES: tuple[Case, ...] = (
    # ---- Llama-3
    _c("llama3_fsdp", "llama3", "llama3_debugmodel", cpu_ok=True, note="FSDP2 over all ranks"),
    _c("llama3_tp", "llama3", "llama3_debugmodel", ("--parallelism.tensor_parallel_degree", "2"), cpu_ok=True),
    _c("llama3_hsdp", "llama3", "llama3_debugmodel",
       ("--parallelism.data_parallel_replicate_degree", "2", "--parallelism.data_parallel_shard_degree", "2"),
       ranks=4, cpu_ok=True),
    _c("llama3_pp", "llama3", "llama3_debugmodel",
       ("--parallelism.pipeline_parallel_degree", "2", "--parallelism.pipeline_parallel_schedule", "1F1B"),
       cpu_ok=True),
    _c("llama3_cp_ulysses", "llama3", "llama3_debugmodel", ("--parallelism.context_parallel_degree", "2"),
       cpu_ok=True),
    _c("llama3_async_tp", "llama3", "llama3_debugmodel",
       ("--parallelism.tensor_parallel_degree", "2", "--parallelism.enable_async_tensor_parallel",
        "--training.local_batch_size", "1"),
       note="fused all-gather→GEMM / GEMM→reduce-scatter kernels over peer memory"),
    _c("llama3_fused_kernels", "llama3", "llama3_debugmodel",
       ("--model_converters.converters", "b200_rms_norm,b200_rope,b200_swiglu,b200_cross_entropy,b200_linear"),
       note="every converter of the headline recipe on the debug model"),
    _c("llama3_peer_memory_fsdp", "llama3", "llama3_debugmodel",
       ("--parallelism.fsdp_reduce_scatter", "peer_memory", "--parallelism.fsdp_all_gather", "peer_memory"),
       note="FSDP2 with the peer-memory reduce-scatter and copy-engine all-gather hooks"),
    _c("llama3_checkpoint_async", "llama3", "llama3_debugmodel",
       ("--checkpoint.enable", "--checkpoint.interval", "2", "--checkpoint.async_mode", "async_with_pinned_mem"),
       cpu_ok=True),
    _c("llama3_swap_optimizer", "llama3", "llama3_debugmodel", ("--optimizer.swap_optimizer",),
       note="AdamW moments in pinned host memory"),
    _c("llama3_fake_backend", "llama3", "llama3_debugmodel", ("--comm.mode", "fake_backend"), ranks=1, cpu_ok=True,
       env=(("NGPU", "8"), ("LOCAL_RANK", "0")), steps=1, note="dry run of an 8-rank job in one process"),
    # ---- DeepSeek-V3 / V3.2 / V4
    _c("deepseek_v3_base", "deepseek_v3", "deepseek_v3_smoketest", cpu_ok=True),
    _c("deepseek_v3_tp", "deepseek_v3", "deepseek_v3_smoketest", ("--parallelism.tensor_parallel_degree", "2"),
       cpu_ok=True),
    _c("deepseek_v3_fsdp_ep", "deepseek_v3", "deepseek_v3_smoketest", ("--parallelism.expert_parallel_degree", "2"),
       cpu_ok=True),
    _c("deepseek_v3_fused_ep", "deepseek_v3", "deepseek_v3_smoketest",
       ("--parallelism.expert_parallel_degree", "2", "--model_converters.converters",
        "b200_rms_norm,b200_rope,b200_gmm,b200_moe_dispatch"),
       note="peer-memory dispatch / combine + grouped tcgen05 GEMMs"),
    _c("deepseek_v32_base", "deepseek_v32", "deepseek_v32_smoketest", cpu_ok=True),
    _c("deepseek_v32_tp", "deepseek_v32", "deepseek_v32_smoketest", ("--parallelism.tensor_parallel_degree", "2"),
       cpu_ok=True),
    _c("deepseek_v32_fsdp_ep", "deepseek_v32", "deepseek_v32_smoketest",
       ("--parallelism.expert_parallel_degree", "2"), cpu_ok=True),
    _c("deepseek_v32_cp", "deepseek_v32", "deepseek_v32_smoketest", ("--parallelism.context_parallel_degree", "2"),
       cpu_ok=True, note="all-gather context parallelism of the shared KV latent"),
    _c("deepseek_v4_base", "deepseek_v4", "deepseek_v4_smoketest", cpu_ok=True),
    _c("deepseek_v4_tp", "deepseek_v4", "deepseek_v4_smoketest", ("--parallelism.tensor_parallel_degree", "2"),
       cpu_ok=True),
    _c("deepseek_v4_fsdp_ep", "deepseek_v4", "deepseek_v4_smoketest",
       ("--parallelism.expert_parallel_degree", "2"), cpu_ok=True),
    _c("deepseek_v4_muon", "deepseek_v4", "deepseek_v4_smoketest", ("--optimizer.name", "Muon"), cpu_ok=True),
    _c("deepseek_v4_compile", "deepseek_v4", "deepseek_v4_smoketest",
       ("--compile.enable", "--compile.backend", "aot_eager"), cpu_ok=True,
       note="per-submodule compile plan around the attention cores and the experts"),
    # ---- Qwen3
    _c("qwen3_base", "qwen3", "qwen3_debugmodel", cpu_ok=True),
    _c("qwen3_moe_ep", "qwen3", "qwen3_debugmodel_moe", ("--parallelism.expert_parallel_degree", "2"), cpu_ok=True),
)

_LOSS = re.compile(r"r0\] .*? step:\s+(\d+)\s+loss:\s+([0-9.eE+-]+|nan|inf)", re.IGNORECASE)
_BENIGN = ("TORCH_NCCL_ASYNC_ERROR_HANDLING", "error_handling", "errors='")


def assess(log: str, returncode: int | None, steps: int) -> tuple[bool, str]:
    """(passed, reason) from the exit code and the text of a run."""
    if returncode is None:
        return False, "timeout"
    if returncode != 0:
        return False, f"exit code {returncode}"
    if "Traceback (most recent call last)" in log:
        return False, "traceback in the log"
    for line in log.splitlines():
        low = line.lower()
        if ("error" in low or "exception" in low) and " info " not in low and not any(b.lower() in low for b in _BENIGN):
            if "warning" in low or re.search(r"\]:?W\d{4} ", line):   # warnings, torch's `W<mmdd>` log lines
                continue
            return False, f"error line: {line.strip()[:160]}"
    seen = _LOSS.findall(log)
    bad = [s for s, v in seen if v.lower() in ("nan", "inf")]
    if bad:
        return False, f"loss is NaN / Inf at step {bad[0]}"
    done = max((int(s) for s, _ in seen), default=0)
    if done < steps:
        return False, f"only {done} of {steps} steps logged"
    return True, f"{done} steps"


def command(case: Case, device: str, port: int, out_dir: str) -> list[str]:
    args = ["--module", case.module, "--config", case.config, "--training.steps", str(case.steps),
            "--metrics.log_freq", "1", "--job.dump_folder", os.path.join(out_dir, case.name), *case.overrides]
    if device == "cpu":
        args += ["--training.dtype", "float32"]
    if case.ranks == 1:
        return [sys.executable, "-m", "titan_b200.entry", *args]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={case.ranks}",
            "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "titan_b200.entry", *args]


def run_case(case: Case, device: str, out_dir: str, port: int, timeout: int) -> dict:
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), OMP_NUM_THREADS="2")
    env.update(dict(case.env))
    if device == "cpu":
        env["CUDA_VISIBLE_DEVICES"] = ""
    cmd = command(case, device, port, out_dir)
    t0 = time.time()
    try:
        res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
        log, rc = res.stdout + res.stderr, res.returncode
    except subprocess.TimeoutExpired as exc:
        log = (exc.stdout or b"").decode(errors="replace") + (exc.stderr or b"").decode(errors="replace") \
            if isinstance(exc.stdout, bytes) or isinstance(exc.stderr, bytes) else (exc.stdout or "") + (exc.stderr or "")
        rc = None
    with open(os.path.join(out_dir, f"{case.name}.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + log)
    ok, why = assess(log, rc, case.steps)
    return {"case": case.name, "status": "passed" if ok else "failed", "reason": why, "ranks": case.ranks,
            "seconds": round(time.time() - t0, 1)}


def visible_gpus() -> int:
    try:
        import torch

        return torch.cuda.device_count()
    except Exception:  # noqa: BLE001
        return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("out_dir")
    ap.add_argument("--case", action="append", default=[], help="run only these cases (repeatable)")
    ap.add_argument("--device", choices=["auto", "cpu", "gpu"], default="auto")
    ap.add_argument("--max-ranks", type=int, default=None, help="skip cases that need more ranks")
    ap.add_argument("--timeout", type=int, default=600, help="seconds per case")
    ap.add_argument("--list", action="store_true")
    args = ap.parse_args(argv)
    if args.list:
        for c in CASES:
            print(f"{c.name:32s} ranks={c.ranks} {'cpu+gpu' if c.cpu_ok else 'gpu'}  {c.note}")
        return 0
    gpus = visible_gpus()
    device = args.device if args.device != "auto" else ("gpu" if gpus > 0 else "cpu")
    os.makedirs(args.out_dir, exist_ok=True)
    known = {c.name for c in CASES}
    for name in args.case:
        if name not in known:
            raise SystemExit(f"unknown case {name!r}; --list shows the table")
    report = []
    for i, case in enumerate(CASES):
        if args.case and case.name not in args.case:
            continue
        limit = args.max_ranks if args.max_ranks is not None else (gpus if device == "gpu" else 4)
        if device == "cpu" and not case.cpu_ok:
            report.append({"case": case.name, "status": "skipped", "reason": "needs a B200"})
        elif case.ranks > limit:
            report.append({"case": case.name, "status": "skipped", "reason": f"needs {case.ranks} ranks"})
        else:
            report.append(run_case(case, device, args.out_dir, 29700 + i, args.timeout))
        print(json.dumps(report[-1]), flush=True)
    with open(os.path.join(args.out_dir, "report.json"), "w") as f:
        json.dump({"device": device, "cases": report}, f, indent=1)
    failed = [r["case"] for r in report if r["status"] == "failed"]
    print(f"{sum(r['status'] == 'passed' for r in report)} passed, {len(failed)} failed, "
          f"{sum(r['status'] == 'skipped' for r in report)} skipped" + (f": {failed}" if failed else ""))
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
