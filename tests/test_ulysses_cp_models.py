"""Ulysses context parallelism at model level on gloo ranks: CP2 resumes from a single-rank checkpoint and must reproduce
the single-rank step, with the exchanges as hooks around the attention core and folded into the projections."""

import pytest

from _launch import launch, step_line


def _common(module, config, folder):
    return ["--module", module, "--config", config, "--training.seq_len", "256", "--comm.backend", "gloo",
            "--training.local_batch_size", "2", "--job.dump_folder", folder, "--checkpoint.enable",
            "--checkpoint.interval", "1", "--training.steps", "2"]


# Qwen3 under CP2 is covered by tests/test_qwen3.py (same two-launch comparison)
@pytest.mark.parametrize("module,config,port", [("llama3", "llama3_debugmodel", 29760)])
def test_cp2_reproduces_single_rank(tmp_path, module, config, port):
    common = _common(module, config, str(tmp_path / "run"))
    ref = step_line(launch(common, 1, port), 2)
    cp = [*common, "--checkpoint.load_step", "1", "--parallelism.data_parallel_shard_degree", "1",
          "--parallelism.context_parallel_degree", "2"]
    hooked = step_line(launch(cp, 2, port + 1), 2)
    fused = step_line(launch([*cp, "--parallelism.context_parallel_fused_projections"], 2, port + 2), 2)
    for got in (hooked, fused):
        assert abs(got[0] - ref[0]) < 2e-3 and abs(got[1] - ref[1]) < 2e-3 * max(ref[1], 1.0), (got, ref)
