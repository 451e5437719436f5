"""HF export of expert weights that are sharded inside the expert (worker: tests/_mp_expert_export_worker.py)."""

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_export_gathers_inner_shards_and_keeps_expert_shards_local():
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29749", os.path.join(ROOT, "tests", "_mp_expert_export_worker.py")]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    log = res.stdout + res.stderr
    assert res.returncode == 0 and "rank 0 ok" in log and "rank 1 ok" in log, log[-5000:]
