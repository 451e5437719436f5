"""Pipeline parallelism on gloo ranks: a two-stage 1F1B run resumes from a single-rank checkpoint and must reproduce the
single-rank step (loss on the last stage, gradient norm everywhere); a 2 x 2 (PP x FSDP) run trains."""

import re

from _launch import launch, step_line

_COMMON = ["--module", "llama3", "--config", "llama3_debugmodel", "--training.seq_len", "128", "--comm.backend", "gloo",
           "--training.local_batch_size", "4"]


def _last_stage_line(log, step):
    rows = re.findall(rf"r\d+\] .*? step:\s+{step}\s+loss:\s+(-?[0-9]+\.[0-9]+)\s+grad_norm:\s+([0-9.]+)", log)
    assert rows, log[-3000:]
    loss, gnorm = max((float(a), float(b)) for a, b in rows)  # stages without the loss log 0 or -1
    return loss, gnorm


def test_pp2_reproduces_single_rank_step(tmp_path):
    folder = str(tmp_path / "run")
    common = [*_COMMON, "--job.dump_folder", folder, "--checkpoint.enable", "--checkpoint.interval", "1",
              "--training.steps", "2"]
    ref = step_line(launch(common, 1, 29700), 2)
    env = {"LOG_RANK": "0,1"}
    log = launch([*common, "--checkpoint.load_step", "1", "--parallelism.data_parallel_shard_degree", "1",
                  "--parallelism.pipeline_parallel_degree", "2", "--parallelism.pipeline_parallel_microbatch_size", "2"],
                 2, 29701, env_extra=env)
    got = _last_stage_line(log, 2)
    assert abs(got[0] - ref[0]) < 2e-3 and abs(got[1] - ref[1]) < 2e-3 * max(ref[1], 1.0), (got, ref)


def test_pp2_with_fsdp2_trains(tmp_path):
    log = launch([*_COMMON, "--job.dump_folder", str(tmp_path / "r"), "--training.steps", "3",
                  "--parallelism.data_parallel_shard_degree", "2", "--parallelism.pipeline_parallel_degree", "2",
                  "--parallelism.pipeline_parallel_microbatch_size", "2"], 4, 29702)
    loss, gnorm = _last_stage_line(log, 3)
    assert 0 < loss < 12 and gnorm == gnorm
