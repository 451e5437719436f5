"""DeepSeek-V4 context parallelism (window exchange + gathered compressed keys) on two gloo ranks.

Models the reference's tests/unit_tests/distributed/test_compressor_attention_cp.py: the sharded run must reproduce
the unsharded step.
"""

import torch

from _launch import launch, step_line


def test_window_exchange_forward_backward_single_rank_is_identity():
    import torch.distributed as dist

    from titan_b200.parallel.context_parallel.compressor_attention_cp import window_exchange

    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29633", rank=0, world_size=1)
    try:
        x = torch.randn(2, 8, 4, requires_grad=True)
        y = window_exchange(x, 4, dist.group.WORLD)
        assert torch.equal(y, x)
        y.sum().backward()
        assert torch.equal(x.grad, torch.ones_like(x))
    finally:
        dist.destroy_process_group()


def test_cp2_reproduces_single_rank_step(tmp_path):
    folder = str(tmp_path / "run")
    common = ["--module", "deepseek_v4", "--config", "deepseek_v4_smoketest", "--training.seq_len", "256",
              "--comm.backend", "gloo", "--training.local_batch_size", "2", "--training.num_mtp_modules", "0",
              "--model_converters.converters", "b200_smla", "--job.dump_folder", folder, "--checkpoint.enable",
              "--checkpoint.interval", "1", "--training.steps", "2"]
    ref = step_line(launch(common, 1, 29630), 2)
    got = step_line(launch([*common, "--checkpoint.load_step", "1", "--parallelism.data_parallel_shard_degree", "1",
                            "--parallelism.context_parallel_degree", "2"], 2, 29631), 2)
    assert abs(got[0] - ref[0]) < 2e-3 and abs(got[1] - ref[1]) < 2e-3 * max(ref[1], 1.0), (got, ref)
