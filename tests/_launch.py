"""Helpers for tests that start the trainer as child processes (CPU, gloo)."""

import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def launch(args, nproc, port, timeout=900, env_extra=None):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "titan_b200.entry", *args]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    log = res.stdout + res.stderr
    assert res.returncode == 0, log[-4000:]
    return log


def losses(log):
    return [float(m) for m in re.findall(r"r0\] .*? step:\s+\d+\s+loss:\s+([0-9.]+|nan|inf)", log)]


def step_line(log, step):
    """(loss, grad_norm) that rank 0 logged for ``step``."""
    m = re.search(rf"r0\] .*? step:\s+{step}\s+loss:\s+([0-9.]+)\s+grad_norm:\s+([0-9.]+)", log)
    assert m, log[-3000:]
    return float(m.group(1)), float(m.group(2))
