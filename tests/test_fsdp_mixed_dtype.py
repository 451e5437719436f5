"""FSDP over a block whose parameters are stored in bf16 except one fp32 module (the lightning indexer's gate
projection): the odd module becomes a parameter group of its own and keeps its dtype."""

import torch
import torch.nn as nn

from _launch import launch, losses


def test_odd_dtype_modules_are_found_by_element_count():
    from titan_b200.parallel.fsdp import _odd_dtype_modules

    block = nn.Sequential(nn.Linear(32, 32), nn.Linear(32, 4), nn.LayerNorm(32)).to(torch.bfloat16)
    block[1].float()
    assert _odd_dtype_modules(block) == [block[1]]
    assert _odd_dtype_modules(block, skip=block[1]) == []
    assert _odd_dtype_modules(nn.Linear(4, 4)) == []


def test_deepseek_v32_bf16_storage_with_fp32_gate_trains_under_fsdp_gloo(tmp_path):
    log = launch(["--module", "deepseek_v32", "--config", "deepseek_v32_smoketest", "--training.steps", "2",
                  "--training.dtype", "bfloat16", "--metrics.log_freq", "1", "--job.dump_folder", str(tmp_path)],
                 nproc=2, port=29812)
    got = losses(log)
    assert len(got) == 2 and all(x == x and x < 20 for x in got), log[-2000:]
