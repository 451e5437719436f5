"""Hardware-free end-to-end tier: Llama-3 debug model, CPU/gloo, world_size=2 FSDP, fp32."""

import os

import torch
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, nproc=2, port=29541, timeout=900, env_extra=None):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    env.update(env_extra or {})
    if nproc == 1:
        cmd = [sys.executable, "-m", "titan_b200.entry", *args]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "titan_b200.entry", *args]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    log = res.stdout + res.stderr
    assert res.returncode == 0, log[-4000:]
    assert "Traceback" not in log, log[-4000:]
    return log


def _losses(log):
    return [float(m) for m in re.findall(r"r0\] .*? step:\s+\d+\s+loss:\s+([0-9.]+|nan|inf)", log)]


def test_llama3_debug_fsdp2_gloo_ten_steps_checkpoint_roundtrip(tmp_path):
    base = ["--module", "llama3", "--config", "llama3_debugmodel", "--job.dump_folder", str(tmp_path),
            "--checkpoint.enable", "--checkpoint.interval", "5", "--debug.seed", "0"]
    log = _run(base + ["--training.steps", "10"])
    losses = _losses(log)
    assert len(losses) == 10 and all(l == l and l < 20 for l in losses)
    assert os.path.exists(tmp_path / "checkpoint" / "step-10" / ".metadata")
    assert os.path.exists(tmp_path / "checkpoint" / "step-5" / ".metadata")
    # resume: the existing step-10 wins, two more steps run (11, 12)
    log2 = _run(base + ["--training.steps", "12"], port=29542)
    assert "loaded checkpoint" in log2 and "training starts at step 11" in log2
    assert len(_losses(log2)) == 2
    # the per-rank token counter continues from the checkpoint: 12 steps x 4 sequences x 512 tokens
    import torch.distributed.checkpoint as dcp

    seen = {"train_state.ntokens_seen": torch.zeros((), dtype=torch.int64)}
    dcp.load(seen, checkpoint_id=str(tmp_path / "checkpoint" / "step-12"))
    assert int(seen["train_state.ntokens_seen"]) == 12 * 4 * 512, seen
    # a checkpoint written by 2 ranks loads into 1 rank (DCP reshards)
    log3 = _run(base + ["--training.steps", "13"], nproc=1)
    assert "training starts at step 13" in log3


def test_deterministic_double_run_is_bitwise_equal(tmp_path):
    common = ["--module", "llama3", "--config", "llama3_debugmodel", "--debug.seed", "1", "--debug.deterministic",
              "--training.seq_len", "128", "--training.local_batch_size", "2", "--training.steps", "3"]
    a = _losses(_run(common + ["--job.dump_folder", str(tmp_path / "a")], nproc=1))
    b = _losses(_run(common + ["--job.dump_folder", str(tmp_path / "b")], nproc=1))
    assert len(a) == 3 and a == b


def test_fake_backend_dry_run_and_simulator(tmp_path):
    log = _run(["--module", "llama3", "--config", "llama3_debugmodel", "--comm.mode", "fake_backend",
                "--job.dump_folder", str(tmp_path)], nproc=1, env_extra={"NGPU": "8"})
    assert "world 8" in log and "dp_shard 8" in log and len(_losses(log)) == 1
    rep = tmp_path / "mem.json"
    log = _run(["--module", "llama3", "--config", "llama3_debugmodel", "--memory_sim.enable",
                "--memory_sim.report_path", str(rep)], nproc=1, env_extra={"NGPU": "2"})
    assert "memory estimate per rank (2 ranks" in log and "FITS" in log and rep.exists()
