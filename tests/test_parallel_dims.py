import pytest

from titan_b200.parallel.parallel_dims import ParallelDims


def test_auto_shard_degree():
    pd = ParallelDims(dp_shard=-1, tp=2, world_size=8)
    assert pd.dp_shard == 4 and pd.fsdp_enabled and pd.tp_enabled and not pd.cp_enabled
    assert pd.non_data_parallel_size == 2 and pd.seq_len_divisor == 4
    assert pd.fsdp_gradient_divide_factor == 4


def test_validation():
    with pytest.raises(ValueError):
        ParallelDims(dp_shard=3, tp=2, world_size=8)
    with pytest.raises(ValueError):
        ParallelDims(dp_shard=-1, tp=3, world_size=8)
    with pytest.raises(ValueError):
        ParallelDims(dp_shard=8, ep=3, world_size=8)
    with pytest.raises(ValueError):
        ParallelDims(dp_shard=4, tp=2, ep=2, etp=4, world_size=8)


def test_ep_sizes():
    pd = ParallelDims(dp_shard=8, ep=8, world_size=8)
    assert pd.efsdp == 1
    pd = ParallelDims(dp_shard=4, tp=2, ep=4, etp=2, world_size=8)
    assert pd.efsdp == 1
    pd = ParallelDims(dp_shard=4, tp=2, ep=8, etp=1, world_size=8)  # tp ranks borrowed by ep
    assert pd.efsdp == 1
    pd = ParallelDims(dp_shard=2, cp=2, tp=2, ep=2, etp=2, world_size=8)
    assert pd.efsdp == 2


def test_coordinates_cover_world():
    pd = ParallelDims(dp_replicate=2, dp_shard=2, tp=2, world_size=8)
    seen = {tuple(sorted(pd.coordinate(r).items())) for r in range(8)}
    assert len(seen) == 8
    assert pd.coordinate(5) == {"tp": 1, "cp": 0, "dp_shard": 0, "dp_replicate": 1, "pp": 0}


def test_single_rank_mesh(gloo_single_rank):
    pd = ParallelDims(dp_shard=1, world_size=1)
    pd.build_mesh("cpu")
    assert pd.get_optional_mesh("tp") is None and pd.get_optional_mesh("fsdp") is None
    with pytest.raises(ValueError):
        pd.get_mesh("tp")


def test_single_process_without_a_process_group_hands_out_no_mesh():
    import torch.distributed as dist

    if dist.is_initialized():
        pytest.skip("a process group exists in this interpreter")
    pd = ParallelDims(dp_shard=-1, world_size=1)
    assert pd.get_optional_mesh("tp") is None and pd.get_optional_mesh("fsdp") is None
    assert pd.mesh_even_if_trivial("efsdp") is None
    assert not dist.is_initialized()   # asking did not try to create one
