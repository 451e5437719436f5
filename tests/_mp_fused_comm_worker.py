"""Worker of the multi-GPU fused-collective tests (launched by torch.distributed.run)."""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from titan_b200.ops import _lib, fused_comm

    group = dist.group.WORLD
    torch.manual_seed(1234 + rank)
    dev = "cuda"
    for rep in range(3):  # repetition exercises slot reuse and epoch progress
        m_shard, K, N = 256, 512, 768
        a = torch.randn(m_shard, K, device=dev, dtype=torch.bfloat16)
        torch.manual_seed(7)
        b = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        torch.manual_seed(1234 + rank + rep)
        out = fused_comm.all_gather_matmul(a, b, group)
        ref = fused_comm.all_gather_matmul_baseline(a, b, group)
        torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)

        n_shard = 256
        w = (torch.randn(n_shard, K, device=dev) * 0.05).to(torch.bfloat16)
        torch.manual_seed(11)
        x = torch.randn(384, K, device=dev, dtype=torch.bfloat16)
        torch.manual_seed(1234 + rank + rep)
        out = fused_comm.all_gather_weight_matmul(x, w, group)
        full = torch.empty(world * n_shard, K, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, w, group=group)
        torch.testing.assert_close(out.float(), (x @ full.t()).float(), rtol=2e-2, atol=2e-2)

        M = 128 * world * 2
        a2 = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        b2 = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        out = fused_comm.matmul_reduce_scatter(a2, b2, group)
        ref = fused_comm.matmul_reduce_scatter_baseline(a2, b2, group)
        torch.testing.assert_close(out.float(), ref.float(), rtol=3e-2, atol=6e-2)

        bucket = torch.randn(world * 4096 + 0, device=dev).to(torch.bfloat16)
        out = fused_comm.castscale_reduce_scatter(bucket, 1.0 / world, torch.float32, group)
        ref = fused_comm.castscale_reduce_scatter_baseline(bucket, 1.0 / world, torch.float32, group)
        torch.testing.assert_close(out, ref, rtol=1e-3, atol=1e-3)
    torch.cuda.synchronize()
    _lib.shared_status().raise_if_set("fused comm")

    # expert-parallel fused MoE against the single-rank fused MoE with all experts
    from titan_b200.converters.gmm import FusedGroupedExperts
    from titan_b200.ops import moe, moe_comm

    E, D, H, T, k = 8 * world if world <= 2 else 8, 256, 128, 512, 2
    torch.manual_seed(99)
    full = FusedGroupedExperts(D, H, E).to(dev).bfloat16()
    full.init_states()
    e_local = E // world
    local = FusedGroupedExperts(D, H, e_local).to(dev).bfloat16()
    with torch.no_grad():
        local.w13.copy_(full.w13[rank * e_local:(rank + 1) * e_local])
        local.w2.copy_(full.w2[rank * e_local:(rank + 1) * e_local])
    local.num_experts = E
    torch.manual_seed(500 + rank)
    x = torch.randn(T, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    logits = torch.randn(T, E, device=dev)
    gate, idx, _ = moe.router_topk(logits, k, score_func="softmax")
    gate = gate.detach().requires_grad_()
    out = moe_comm.moe_forward_ep(x, gate, idx, local, group, base=None, score_before_experts=False)
    plan = moe.make_plan(idx, E)
    xr = x.detach().clone().requires_grad_()
    gr = gate.detach().clone().requires_grad_()
    ref = moe.combine(full.forward_padded(moe.permute(xr, plan), plan.offs), plan, T, weights=gr)
    torch.testing.assert_close(out.float(), ref.float(), rtol=3e-2, atol=3e-2)
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g)
    torch.testing.assert_close(x.grad.float(), xr.grad.float(), rtol=5e-2, atol=5e-2)
    torch.testing.assert_close(gate.grad, gr.grad, rtol=5e-2, atol=0.3)
    # expert weight grads: each rank holds grads of its experts from ALL ranks' tokens
    gw = full.w2.grad.float().clone()
    dist.all_reduce(gw, group=group)
    torch.testing.assert_close(local.w2.grad.float(), gw[rank * e_local:(rank + 1) * e_local], rtol=5e-2, atol=0.3)
    torch.cuda.synchronize()
    _lib.shared_status().raise_if_set("moe ep")

    # Ulysses: projection fused with the head->sequence exchange and the way back, forward and backward,
    # against all_to_all_single + matmul
    from titan_b200.ops import ulysses_fused as uf

    for rep in range(3):
        batch, s_loc, dim, heads, hd = 2, 256, 512, 4 * world, 64
        nq = heads * hd
        torch.manual_seed(99)
        wq = (torch.randn(nq, dim, device=dev) * 0.05).to(torch.bfloat16)
        wo = (torch.randn(dim, nq, device=dev) * 0.05).to(torch.bfloat16)
        torch.manual_seed(4321 + rank + rep)
        x = torch.randn(batch * s_loc, dim, device=dev, dtype=torch.bfloat16)
        xa, wqa, woa = (t.clone().requires_grad_(True) for t in (x, wq, wo))
        xb, wqb, wob = (t.clone().requires_grad_(True) for t in (x, wq, wo))
        q = uf.proj_all_to_all(xa, wqa, s_loc, group)           # [batch * s_full, nq / world]
        y = uf.all_to_all_proj(torch.tanh(q), woa, s_loc, group)  # [batch * s_loc, dim]
        # differentiable reference: matmul + the autograd all-to-all of the hook-based Ulysses path
        from titan_b200.parallel.context_parallel.ulysses import all_to_all_4d

        qr = all_to_all_4d((xb @ wqb.t()).view(batch, s_loc, world, -1), 2, 1, group).reshape(batch * s_loc * world, -1)
        o4 = torch.tanh(qr).view(batch, s_loc * world, 1, -1)
        yr = all_to_all_4d(o4, 1, 2, group).reshape(batch * s_loc, -1) @ wob.t()
        torch.testing.assert_close(q.float(), qr.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(y.float(), yr.float(), rtol=3e-2, atol=3e-2)
        gy = torch.randn_like(y)
        y.backward(gy)
        yr.backward(gy)
        torch.testing.assert_close(xa.grad.float(), xb.grad.float(), rtol=5e-2, atol=5e-2)
        torch.testing.assert_close(wqa.grad.float(), wqb.grad.float(), rtol=5e-2, atol=0.3)
        torch.testing.assert_close(woa.grad.float(), wob.grad.float(), rtol=5e-2, atol=0.3)
    torch.cuda.synchronize()
    _lib.shared_status().raise_if_set("ulysses fused")
    dist.barrier()
    if rank == 0:
        print("FUSED_COMM_WORKER_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
