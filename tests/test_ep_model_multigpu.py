"""Expert parallelism at model level on 2 GPUs.  One GPU trains two steps on a global batch of 2 rows and checkpoints
after the first; two GPUs (EP2 x FSDP2, one row each from the same global stream) resume there and must log the same
step-2 loss and gradient norm.  Run for the plain path (NCCL all-to-all around `torch._grouped_mm`) and for the fused
path (grouped-GEMM experts + peer-memory dispatch / combine): this pins the gradient scaling of the expert weights
(FSDP's divide factor has to reach them) as well as the exchange itself."""

import pytest
import torch

from _launch import launch, step_line

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

_COMMON = ["--module", "deepseek_v3", "--config", "deepseek_v3_debugmodel", "--training.seq_len", "512",
           "--training.dtype", "bfloat16", "--training.steps", "2", "--optimizer.implementation", "fused",
           "--dataloader.global_stream", "--checkpoint.enable", "--checkpoint.interval", "1",
           "--debug.grad_norm_breakdown"]
_FUSED = ["--model_converters.converters", "b200_moe_dispatch,b200_gmm"]


@pytest.mark.parametrize("name,extra,port", [("plain", [], 29720), ("fused", _FUSED, 29730)])
def test_ep2_reproduces_single_gpu_step(tmp_path, name, extra, port):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = {"NCCL_NVLS_ENABLE": "0", "TORCH_SYMM_MEM_DISABLE_MULTICAST": "1"}
    common = [*_COMMON, *extra, "--job.dump_folder", str(tmp_path / name)]
    one = launch([*common, "--training.local_batch_size", "2"], 1, port, env_extra=env)
    two = launch([*common, "--training.local_batch_size", "1", "--checkpoint.load_step", "1",
                  "--parallelism.data_parallel_shard_degree", "2", "--parallelism.expert_parallel_degree", "2",
                  *(["--parallelism.expert_parallel_comm_backend", "fused_p2p"] if extra else [])],
                 2, port + 1, env_extra=env)
    ref, got = step_line(one, 2), step_line(two, 2)
    detail = [ln for ln in (one + two).splitlines() if "grad norm of" in ln]
    assert abs(got[0] - ref[0]) < 2e-2 * max(1.0, abs(ref[0])), (ref, got, detail)
    assert abs(got[1] - ref[1]) < 3e-2 * max(1.0, ref[1]), (ref, got, detail)
