"""Expert parallelism at model level on 2 GPUs: the fused path (grouped-GEMM experts + peer-memory dispatch / combine)
must train like the plain path (NCCL all-to-all around `torch._grouped_mm`): same loss and the same gradient norm on the
same data, which also pins the gradient scaling of the expert weights (FSDP's divide factor has to reach them)."""

import pytest
import torch

from _launch import launch, step_line

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

_COMMON = ["--module", "deepseek_v3", "--config", "deepseek_v3_debugmodel", "--training.seq_len", "512",
           "--training.local_batch_size", "2", "--training.dtype", "bfloat16", "--training.steps", "3",
           "--parallelism.expert_parallel_degree", "2", "--optimizer.implementation", "fused"]


def test_fused_ep2_matches_nccl_ep2(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = {"NCCL_NVLS_ENABLE": "0", "TORCH_SYMM_MEM_DISABLE_MULTICAST": "1"}
    plain = launch([*_COMMON, "--job.dump_folder", str(tmp_path / "a")], 2, 29720, env_extra=env)
    fused = launch([*_COMMON, "--job.dump_folder", str(tmp_path / "b"), "--model_converters.converters",
                    "b200_moe_dispatch,b200_gmm", "--parallelism.expert_parallel_comm_backend", "fused_p2p"],
                   2, 29721, env_extra=env)
    for step in (1, 2, 3):
        a, b = step_line(plain, step), step_line(fused, step)
        assert abs(a[0] - b[0]) < 3e-2 * max(1.0, abs(a[0])), (step, a, b)
        assert abs(a[1] - b[1]) < 5e-2 * max(1.0, a[1]), (step, a, b)
