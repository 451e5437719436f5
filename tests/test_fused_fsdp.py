"""Fused-collective FSDP linears (through the library fallbacks of the fused ops on CPU): a two-rank run that resumes
from an FSDP2 checkpoint must reproduce FSDP2's next step; the checkpoint written by the fused layout loads back."""

from _launch import launch, step_line


def test_fused_fsdp_reproduces_fsdp2_step(tmp_path):
    folder = str(tmp_path / "run")
    common = ["--module", "llama3", "--config", "llama3_debugmodel", "--training.seq_len", "256", "--comm.backend",
              "gloo", "--training.local_batch_size", "1", "--job.dump_folder", folder, "--checkpoint.enable",
              "--checkpoint.interval", "1", "--training.steps", "2"]
    ref = step_line(launch(common, 2, 29670), 2)
    got = step_line(launch([*common, "--checkpoint.load_step", "1", "--parallelism.fsdp_fused_collectives"], 2, 29671), 2)
    assert abs(got[0] - ref[0]) < 2e-3 and abs(got[1] - ref[1]) < 2e-3 * max(ref[1], 1.0), (got, ref)
    # the fused layout saved step 2; plain FSDP2 continues from it
    nxt = launch([*common, "--training.steps", "3", "--checkpoint.load_step", "2"], 2, 29672)
    assert step_line(nxt, 3)[0] < 12
