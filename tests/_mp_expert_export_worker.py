"""Two gloo ranks: HF export of stacked expert weights that are sharded over the expert dim, inside the expert, or
both ways on a 2-D mesh.  Run by tests/test_expert_export_sharded.py."""

import sys

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.tensor import Replicate, Shard, distribute_tensor

from titan_b200.models.deepseek_v3.state_dict_adapter import MoEStateDictAdapter


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    full = torch.randn(4, 6, 8)   # [experts, rows, columns]
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("x",))
    for placement in (Shard(0), Shard(1), Shard(2), Replicate()):
        first, n, local = MoEStateDictAdapter._local_expert_range(distribute_tensor(full.clone(), mesh, [placement]))
        if isinstance(placement, Shard) and placement.dim == 0:
            assert (first, n) == (rank * 4 // world, 4 // world), (placement, first, n)
        else:
            assert (first, n) == (0, 4), (placement, first, n)   # inner shards are gathered: whole experts
        torch.testing.assert_close(local, full[first:first + n])
    mesh2 = init_device_mesh("cpu", (world, 1), mesh_dim_names=("e", "t"))
    first, n, local = MoEStateDictAdapter._local_expert_range(
        distribute_tensor(full.clone(), mesh2, [Shard(0), Shard(2)]))
    assert (first, n) == (rank * 4 // world, 4 // world)
    torch.testing.assert_close(local, full[first:first + n])
    dist.destroy_process_group()
    print(f"rank {rank} ok")


if __name__ == "__main__":
    sys.exit(main())
