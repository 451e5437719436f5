"""Fused sequence-parallel linears: autograd identities on one rank, and a two-rank run through the library fallbacks
of the fused ops (same dataflow as on GPUs) that must reproduce the single-rank step."""

import torch
import torch.distributed as dist

from _launch import launch, step_line


def test_ag_multi_linear_and_linear_rs_gradients_single_rank():
    from titan_b200.parallel.async_tp import ag_multi_linear, linear_rs

    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29653", rank=0, world_size=1)
    try:
        g = dist.group.WORLD
        torch.manual_seed(0)
        x = torch.randn(16, 32, requires_grad=True)
        wa, wb = torch.randn(24, 32, requires_grad=True), torch.randn(8, 32, requires_grad=True)
        wo = torch.randn(32, 24, requires_grad=True)
        a, b = ag_multi_linear(x, [wa, wb], g)
        y = linear_rs(torch.tanh(a), wo, g) + b.sum(dim=1, keepdim=True)
        y.pow(2).sum().backward()
        xr, war, wbr, wor = (t.detach().clone().requires_grad_() for t in (x, wa, wb, wo))
        yr = torch.tanh(xr @ war.t()) @ wor.t() + (xr @ wbr.t()).sum(dim=1, keepdim=True)
        yr.pow(2).sum().backward()
        for got, ref in ((x, xr), (wa, war), (wb, wbr), (wo, wor)):
            assert torch.allclose(got.grad, ref.grad, atol=1e-4, rtol=1e-4)
    finally:
        dist.destroy_process_group()


def test_async_tp2_reproduces_single_rank_step(tmp_path):
    """Two sequences per rank: the fused operators run once per sequence (a single sequence is the same call without
    the stacking; the other-model cases below use it)."""
    folder = str(tmp_path / "run")
    common = ["--module", "llama3", "--config", "llama3_debugmodel", "--training.seq_len", "256", "--comm.backend",
              "gloo", "--training.local_batch_size", "2", "--job.dump_folder", folder, "--checkpoint.enable",
              "--checkpoint.interval", "1", "--training.steps", "2"]
    ref = step_line(launch(common, 1, 29650), 2)
    got = step_line(launch([*common, "--checkpoint.load_step", "1", "--parallelism.data_parallel_shard_degree", "1",
                            "--parallelism.tensor_parallel_degree", "2",
                            "--parallelism.enable_async_tensor_parallel"], 2, 29651), 2)
    assert abs(got[0] - ref[0]) < 2e-3 and abs(got[1] - ref[1]) < 2e-3 * max(ref[1], 1.0), (got, ref)


import pytest


@pytest.mark.parametrize("module,config,port", [("deepseek_v3", "deepseek_v3_debugmodel", 29655),
                                                ("qwen3", "qwen3_debugmodel", 29658)])
def test_async_tp_fuses_row_parallel_linears_of_other_models(tmp_path, module, config, port):
    """The model-independent half of async TP (GEMM -> reduce-scatter for every row-parallel linear that returns to
    the sequence shard) on an MLA + MoE model and on Qwen3: a TP2 run with the switch on reproduces one rank."""
    folder = str(tmp_path / "run")
    common = ["--module", module, "--config", config, "--training.seq_len", "128", "--comm.backend", "gloo",
              "--training.local_batch_size", "1", "--job.dump_folder", folder, "--checkpoint.enable",
              "--checkpoint.interval", "1", "--training.steps", "2"]
    ref = step_line(launch(common, 1, port), 2)
    log = launch([*common, "--checkpoint.load_step", "1", "--parallelism.data_parallel_shard_degree", "1",
                  "--parallelism.tensor_parallel_degree", "2", "--parallelism.enable_async_tensor_parallel"], 2,
                 port + 1)
    got = step_line(log, 2)
    assert abs(got[0] - ref[0]) < 2e-3 and abs(got[1] - ref[1]) < 2e-3 * max(ref[1], 1.0), (got, ref)


def test_tcgen05_linear_converter_keeps_tensor_parallel_semantics(tmp_path):
    """`b200_linear` under TP2 multiplies the local shards itself (column shard -> Shard(-1), row shard -> Partial):
    the step has to equal the single-rank step (on CPU the local products run through the library)."""
    folder = str(tmp_path / "run")
    common = ["--module", "llama3", "--config", "llama3_debugmodel", "--training.seq_len", "128", "--comm.backend",
              "gloo", "--training.local_batch_size", "2", "--job.dump_folder", folder, "--checkpoint.enable",
              "--checkpoint.interval", "1", "--training.steps", "2", "--model_converters.converters", "b200_linear"]
    ref = step_line(launch(common, 1, 29661), 2)
    got = step_line(launch([*common, "--checkpoint.load_step", "1", "--parallelism.data_parallel_shard_degree", "1",
                            "--parallelism.tensor_parallel_degree", "2"], 2, 29662), 2)
    assert abs(got[0] - ref[0]) < 2e-3 and abs(got[1] - ref[1]) < 2e-3 * max(ref[1], 1.0), (got, ref)
