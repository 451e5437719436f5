"""Ulysses projections with the exchange folded in: semantics and gradients on gloo ranks (the all-to-all form that
backs the kernels on machines without CUDA) against the dense computation on the whole sequence."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4])
def test_projection_exchange_matches_dense(world):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29740 + world),
           os.path.join(ROOT, "tests", "_mp_ulysses_worker.py")]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    log = res.stdout + res.stderr
    assert res.returncode == 0 and "ULYSSES_WORKER_OK" in log, log[-4000:]
