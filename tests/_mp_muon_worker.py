"""Four gloo ranks: distributed Muon on matrices sharded by FSDP x TP (both layouts of a tensor-parallel linear) and by
HSDP must produce the update of a single-process Muon on the whole matrices.  Run by tests/test_muon_distributed.py."""

import sys

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.tensor import Replicate, Shard, distribute_tensor

from titan_b200.optim.muon import DistributedMuon, SwapDistributedMuon


def run(mesh_shape, names, layouts, cls, **kw):
    torch.manual_seed(0)
    shapes = {"col.weight": (16, 8), "row.weight": (8, 16), "third.weight": (12, 8)}
    full_w = {n: torch.randn(s) for n, s in shapes.items()}
    full_g = [{n: torch.randn(s) for n, s in shapes.items()} for _ in range(2)]
    # reference: one process, whole matrices
    ref_p = [nn.Parameter(full_w[n].clone()) for n in shapes]
    ref = DistributedMuon(ref_p, list(shapes), lr=0.05, weight_decay=0.01)
    for g in full_g:
        for p, n in zip(ref_p, shapes):
            p.grad = g[n].clone()
        ref.step()
    mesh = init_device_mesh("cpu", mesh_shape, mesh_dim_names=names)
    ps = [nn.Parameter(distribute_tensor(full_w[n].clone(), mesh, layouts[n])) for n in shapes]
    opt = cls(ps, list(shapes), lr=0.05, weight_decay=0.01, **kw)
    for g in full_g:
        for p, n in zip(ps, shapes):
            p.grad = distribute_tensor(g[n].clone(), mesh, layouts[n])
        opt.step()
    for p, r, n in zip(ps, ref_p, shapes):
        # the exchange moves bf16 shards; the reference ran Newton-Schulz in bf16 as well
        torch.testing.assert_close(p.full_tensor(), r.detach(), rtol=2e-2, atol=2e-3, msg=lambda m, n=n: f"{n}: {m}")
    return opt


def main():
    dist.init_process_group("gloo")
    tp_layouts = {"col.weight": [Shard(0), Shard(0)], "row.weight": [Shard(0), Shard(1)],
                  "third.weight": [Shard(0), Shard(0)]}
    opt = run((2, 2), ("fsdp", "tp"), tp_layouts, DistributedMuon)
    assert opt.comm_calls > 0
    hsdp = {n: [Replicate(), Shard(0)] for n in tp_layouts}
    opt = run((2, 2), ("dp_replicate", "fsdp"), hsdp, DistributedMuon, extra_reduce_for_hsdp=True)
    run((2, 2), ("fsdp", "tp"), tp_layouts, SwapDistributedMuon, swap_merge_buckets=1)
    dist.barrier()
    if dist.get_rank() == 0:
        print("MUON_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
