"""MoE block under tensor parallelism on two gloo ranks: output, input gradient and parameter gradients equal the
unsharded block for tensor-parallel experts (also with the fused w13 weight) and for expert parallelism that borrows
the tensor-parallel ranks (sequence-sharded tokens)."""

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_moe_block_tp_and_tp_ep_match_unsharded():
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29741", os.path.join(ROOT, "tests", "_mp_moe_tp_worker.py")]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    log = res.stdout + res.stderr
    assert res.returncode == 0 and "MOE_TP_WORKER_OK" in log, log[-5000:]
