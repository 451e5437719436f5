"""Distributed Muon over FSDP x TP and HSDP meshes on four gloo ranks (worker: tests/_mp_muon_worker.py)."""

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_muon_matches_single_process_on_2d_meshes():
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", "29747", os.path.join(ROOT, "tests", "_mp_muon_worker.py")]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    log = res.stdout + res.stderr
    assert res.returncode == 0 and "MUON_WORKER_OK" in log, log[-5000:]
