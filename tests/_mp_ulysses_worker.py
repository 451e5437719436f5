"""Worker (gloo, CPU): Ulysses projections with the fused exchange against the dense single-process computation."""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    from titan_b200.ops import ulysses_fused as uf

    group = dist.group.WORLD
    batch, s_loc, dim, heads, hd = 2, 8, 16, 2 * world, 4
    s_full, nq = s_loc * world, heads * hd
    torch.manual_seed(0)
    x_full = torch.randn(batch, s_full, dim, dtype=torch.float64, requires_grad=True)
    wq = torch.randn(nq, dim, dtype=torch.float64, requires_grad=True)
    wo = torch.randn(dim, nq, dtype=torch.float64, requires_grad=True)
    gy_full = torch.randn(batch, s_full, dim, dtype=torch.float64)
    q_full = x_full @ wq.t()
    y_full = torch.tanh(q_full) @ wo.t()
    (y_full * gy_full).sum().backward()

    sl = slice(rank * s_loc, (rank + 1) * s_loc)
    x = x_full.detach()[:, sl].reshape(batch * s_loc, dim).clone().requires_grad_(True)
    wq_l, wo_l = wq.detach().clone().requires_grad_(True), wo.detach().clone().requires_grad_(True)
    q = uf.proj_all_to_all(x, wq_l, s_loc, group)
    n = nq // world
    torch.testing.assert_close(q.view(batch, s_full, n), q_full.detach()[..., rank * n:(rank + 1) * n])
    y = uf.all_to_all_proj(torch.tanh(q), wo_l, s_loc, group)
    torch.testing.assert_close(y.view(batch, s_loc, dim), y_full.detach()[:, sl])
    (y.view(batch, s_loc, dim) * gy_full[:, sl]).sum().backward()
    torch.testing.assert_close(x.grad.view(batch, s_loc, dim), x_full.grad[:, sl])
    for local, dense in ((wq_l, wq), (wo_l, wo)):
        g = local.grad.clone()
        dist.all_reduce(g, group=group)
        torch.testing.assert_close(g, dense.grad)
    dist.barrier()
    if rank == 0:
        print("ULYSSES_WORKER_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
