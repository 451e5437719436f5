"""Failure detection without faulting anything: failures are made on the host (a rank that leaves, a damaged
checkpoint, an exception inside a step), device waits are bounded and report a status the host reads.

Models the plan of the reference's failure tooling (flight-recorder wiring, crash handling with `trainer.close()`,
transactional optimizer loads) with injected failures instead of real faults.
"""

import os
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_rank_that_leaves_is_detected_by_a_short_process_group_timeout(tmp_path):
    """Rank 1 exits between steps; rank 0's next collective ends with an error within the group's timeout."""
    script = tmp_path / "w.py"
    script.write_text(textwrap.dedent('''
        import datetime, os, sys, time, torch, torch.distributed as dist
        rank = int(os.environ["RANK"])
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
        x = torch.ones(4)
        dist.all_reduce(x)                      # step 1: both ranks present
        assert x[0].item() == 2
        if rank == 1:
            sys.exit(0)                          # leaves between steps, nothing in flight
        t0 = time.time()
        try:
            dist.all_reduce(x)                   # step 2: the peer is gone
            print("UNDETECTED")
        except Exception as e:                   # connection closed / timeout
            print("DETECTED", type(e).__name__, round(time.time() - t0, 1))
    '''))
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29681", str(script)], env=env,
                         capture_output=True, text=True, timeout=180)
    out = res.stdout + res.stderr
    assert "DETECTED" in out and "UNDETECTED" not in out, out[-2000:]


def test_exception_inside_a_step_closes_the_trainer_and_reraises(tmp_path, monkeypatch):
    from titan_b200 import entry
    from titan_b200.trainer.trainer import Trainer

    closed = []
    monkeypatch.setattr(Trainer, "train_step", lambda self, it: (_ for _ in ()).throw(RuntimeError("injected")))
    orig_close = Trainer.close
    monkeypatch.setattr(Trainer, "close", lambda self: (closed.append(True), orig_close(self))[1])
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    monkeypatch.setenv("MASTER_PORT", "29683")
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    with pytest.raises(RuntimeError, match="injected"):
        entry.main(["--module", "llama3", "--config", "llama3_debugmodel", "--comm.backend", "gloo",
                    "--training.steps", "2", "--job.dump_folder", str(tmp_path)])
    assert closed, "trainer.close() must run when a step raises"
    import torch.distributed as dist

    if dist.is_initialized():
        dist.destroy_process_group()


def test_damaged_checkpoint_is_reported_not_half_loaded(tmp_path):
    import torch.distributed.checkpoint as dcp

    state = {"w": torch.arange(1024, dtype=torch.float32), "b": torch.ones(8)}
    path = tmp_path / "step-1"
    dcp.save(state, checkpoint_id=str(path))
    shard = next(p for p in path.iterdir() if p.suffix == ".distcp")
    data = shard.read_bytes()
    shard.write_bytes(data[: len(data) // 3])          # truncated shard
    target = {"w": torch.zeros(1024), "b": torch.zeros(8)}
    from torch.distributed.checkpoint.api import CheckpointException

    with pytest.raises((CheckpointException, Exception)):
        dcp.load(target, checkpoint_id=str(path))
    (path / ".metadata").write_bytes(b"not a pickle")  # corrupt metadata
    with pytest.raises((CheckpointException, Exception)):
        dcp.load({"w": torch.zeros(1024)}, checkpoint_id=str(path))


def test_flight_recorder_env_wiring(tmp_path):
    from titan_b200.config.configs import CommConfig
    from titan_b200.utils.flight_recorder import setup_flight_recorder

    cfg = CommConfig()
    if hasattr(cfg, "trace_buf_size"):
        cfg.trace_buf_size = 2000
    env: dict = {}
    out = setup_flight_recorder(cfg, base_folder=str(tmp_path), env=env)
    assert out is not None
    if getattr(cfg, "trace_buf_size", 0):
        assert env.get("TORCH_NCCL_TRACE_BUFFER_SIZE") == "2000"
        assert env.get("TORCH_NCCL_DUMP_ON_TIMEOUT") in ("1", "true", "True")
        assert str(tmp_path) in env.get("TORCH_NCCL_DEBUG_INFO_TEMP_FILE", "")


@pytest.mark.gpu
def test_device_wait_on_a_flag_nobody_sets_runs_out_and_reports(cuda_device):
    """The wait kernel gives up after its time limit, writes a status code and returns; the context stays usable."""
    import ctypes
    import time

    from titan_b200.ops import _lib

    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.time()
    rc = _lib.lib().tb_wait_flags(flags.data_ptr(), 0, 2, ctypes.c_uint(7), status.data_ptr(), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert status.item() != 0, "an expired wait must leave a status code"
    assert waited < 30
    # the context is alive: ordinary work still runs, and a wait on a flag that IS set returns at once
    flags[:2] = 7
    status.zero_()
    _lib.lib().tb_wait_flags(flags.data_ptr(), 0, 2, ctypes.c_uint(7), status.data_ptr(), _lib.stream_ptr())
    torch.cuda.synchronize()
    assert status.item() == 0 and (torch.ones(4, device="cuda") * 2).sum().item() == 8


def test_kernel_status_word_stops_the_training_loop(tmp_path, monkeypatch):
    """A non-zero kernel status word (here: 'index out of bounds', written by hand into a stand-in word on the host)
    makes the trainer raise at the next log step instead of carrying on with incomplete outputs."""
    from titan_b200 import entry
    from titan_b200.ops._lib import KernelError
    from titan_b200.trainer import kernel_status
    from titan_b200.trainer.trainer import Trainer

    word = torch.zeros(1, dtype=torch.int32)
    orig_init = kernel_status.KernelStatusMonitor.__init__
    monkeypatch.setattr(kernel_status.KernelStatusMonitor, "__init__",
                        lambda self, fn=None: orig_init(self, lambda: word))
    orig_step = Trainer.train_step
    steps = []

    def step(self, it):
        steps.append(self.step)
        if self.step == 2:
            word.fill_(6)   # what a kernel would have written
        return orig_step(self, it)

    monkeypatch.setattr(Trainer, "train_step", step)
    for k, v in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29684"), ("RANK", "0"), ("WORLD_SIZE", "1")):
        monkeypatch.setenv(k, v)
    with pytest.raises(KernelError, match="index out of bounds"):
        entry.main(["--module", "llama3", "--config", "llama3_debugmodel", "--comm.backend", "gloo",
                    "--training.steps", "6", "--metrics.log_freq", "4", "--job.dump_folder", str(tmp_path)])
    assert steps[-1] <= 3, steps   # seen by the non-blocking poll one step later, well before the log step
    assert int(word.item()) == 0   # the word is cleared when it is reported
    import torch.distributed as dist

    if dist.is_initialized():
        dist.destroy_process_group()
