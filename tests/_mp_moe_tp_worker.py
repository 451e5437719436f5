"""Two gloo ranks: an MoE block under tensor / expert parallelism must reproduce the unsharded block (output, input
gradient and every parameter gradient).  Weights are initialised with std 0.3 so that the routed experts carry a
large share of the output.  Run by tests/test_moe_tp.py through torch.distributed.run."""

import sys

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.tensor import DTensor, Shard, distribute_tensor

from titan_b200.models.common.moe import MoE, MoEArgs
from titan_b200.parallel.moe_parallelize import apply_moe_ep_tp


class Block(nn.Module):
    moe_enabled = True

    def __init__(self, moe):
        super().__init__()
        self.moe = moe

    def forward(self, x):
        return self.moe(x)


class Model(nn.Module):
    def __init__(self, moe):
        super().__init__()
        self.layers = nn.ModuleDict({"0": Block(moe)})

    def forward(self, x):
        return self.layers["0"](x)


def build(score_before: bool, fused_w13: bool):
    torch.manual_seed(1234)
    args = MoEArgs(num_experts=4, num_shared_experts=1, top_k=2, score_func="softmax", route_norm=True,
                   score_before_experts=score_before, use_grouped_mm=False, load_balance_coeff=None)
    moe = MoE(32, 48, args)
    for p in moe.parameters():
        nn.init.normal_(p, std=0.3)
    if fused_w13:
        from titan_b200.converters.gmm import FusedGroupedExperts

        old = moe.experts
        new = FusedGroupedExperts(32, 48, 4)
        with torch.no_grad():
            new.w13.copy_(torch.cat([old.w1, old.w3], dim=1))
            new.w2.copy_(old.w2)
        moe.experts = new
    return Model(moe)


def full(t):
    return t.full_tensor() if isinstance(t, DTensor) else t


def grads_by_name(model, fused_w13, world):
    out = {}
    for n, p in model.named_parameters():
        g = p.grad
        if g is None:
            continue
        if isinstance(g, DTensor) and fused_w13 and n.endswith("w13") and any(
                isinstance(pl, Shard) and pl.dim == 1 for pl in g.placements):
            # ranks hold [w1_shard | w3_shard]: undo the interleave for the comparison
            loc = g.to_local()
            h = loc.shape[1] // 2
            parts = [torch.zeros_like(loc) for _ in range(world)]
            dist.all_gather(parts, loc.contiguous())
            g = torch.cat([torch.cat([q[:, :h] for q in parts], 1), torch.cat([q[:, h:] for q in parts], 1)], 1)
        out[n] = full(g)
    return out


def run_case(mode: str, score_before: bool, fused_w13: bool):
    rank, world = dist.get_rank(), dist.get_world_size()
    ref = build(score_before, fused_w13)
    par = build(score_before, fused_w13)
    torch.manual_seed(7)
    x_full = torch.randn(2, 8, 32)
    g_full = torch.randn(2, 8, 32)

    xr = x_full.clone().requires_grad_()
    yr = ref(xr)
    yr.backward(g_full)

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("tp",))
    if mode == "tp":
        apply_moe_ep_tp(par, tp_mesh=mesh)
    elif mode == "tp_ep":   # expert parallelism borrows the tp ranks: tokens stay sequence-sharded
        apply_moe_ep_tp(par, tp_mesh=mesh, ep_mesh=mesh)
    else:
        raise SystemExit(mode)
    xs = distribute_tensor(x_full, mesh, [Shard(1)]).to_local().clone().requires_grad_()
    xd = DTensor.from_local(xs, mesh, [Shard(1)])
    yd = par(xd)
    if not isinstance(yd, DTensor):   # the block hands back this rank's sequence slice
        yd = DTensor.from_local(yd, mesh, [Shard(1)])
    assert yd.placements == (Shard(1),), yd.placements
    y = yd.full_tensor()
    torch.testing.assert_close(y, yr, rtol=1e-4, atol=1e-4)
    gd = distribute_tensor(g_full, mesh, [Shard(1)])
    yd.backward(gd)
    gx = DTensor.from_local(xs.grad, mesh, [Shard(1)]).full_tensor()
    torch.testing.assert_close(gx, xr.grad, rtol=1e-4, atol=1e-4)
    gp, gr = grads_by_name(par, fused_w13, world), grads_by_name(ref, fused_w13, world)
    assert set(gp) == set(gr), (sorted(gp), sorted(gr))
    for n in gr:
        torch.testing.assert_close(gp[n], gr[n], rtol=1e-4, atol=1e-4, msg=lambda m, n=n: f"{mode} {n}: {m}")
    if rank == 0:
        print(f"MOE_TP_CASE_OK {mode} score_before={score_before} fused_w13={fused_w13}", flush=True)


def main():
    dist.init_process_group("gloo")
    for mode in ("tp", "tp_ep"):
        for score_before in (True, False):
            run_case(mode, score_before, False)
    run_case("tp", True, True)
    dist.barrier()
    if dist.get_rank() == 0:
        print("MOE_TP_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
