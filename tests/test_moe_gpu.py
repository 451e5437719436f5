"""MoE kernels (router top-k, padded permutation, grouped tcgen05 GEMM) against PyTorch fp32 references."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_cuda(cuda_device):
    torch.manual_seed(0)


@pytest.mark.parametrize("score_func", ["sigmoid", "softmax", "sqrtsoftplus"])
@pytest.mark.parametrize("E,k", [(64, 6), (8, 2), (256, 8)])
def test_router_topk(score_func, E, k):
    from titan_b200.ops.moe import router_topk, router_topk_ref

    T = 777
    logits = torch.randn(T, E, device="cuda", requires_grad=True)
    bias = torch.randn(E, device="cuda") * 0.1
    gate, idx, counts = router_topk(logits, k, bias=bias, score_func=score_func, route_norm=True, route_scale=2.5)
    lr = logits.detach().clone().requires_grad_()
    g_ref, i_ref, c_ref = router_topk_ref(lr, k, bias=bias, score_func=score_func, route_norm=True, route_scale=2.5)
    assert torch.equal(idx.sort(-1)[0], i_ref.sort(-1)[0])
    torch.testing.assert_close(gate.gather(1, idx.argsort(-1)), g_ref.gather(1, i_ref.argsort(-1)), rtol=1e-4, atol=1e-5)
    assert torch.equal(counts.long(), c_ref.long())
    w = torch.randn_like(gate)
    (gate * w).sum().backward()
    # reference gradient with the SAME slot order as the kernel
    g2 = router_topk_ref(lr, k, bias=bias, score_func=score_func, route_norm=True, route_scale=2.5, forced_idx=idx)[0]
    (g2 * w).sum().backward()
    torch.testing.assert_close(logits.grad, lr.grad, rtol=1e-3, atol=1e-5)


def test_router_forced_idx_hash_routing():
    from titan_b200.ops.moe import router_topk

    T, E, k = 100, 16, 4
    logits = torch.randn(T, E, device="cuda")
    forced = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)])
    gate, idx, counts = router_topk(logits, k, forced_idx=forced, score_func="sigmoid")
    assert torch.equal(idx, forced)
    torch.testing.assert_close(gate, torch.sigmoid(logits).gather(1, forced), rtol=1e-5, atol=1e-6)
    assert int(counts.sum()) == T * k


@pytest.mark.parametrize("T,k,E,D", [(1000, 6, 64, 256), (33, 2, 8, 128), (4096, 6, 64, 2048)])
def test_plan_permute_combine(T, k, E, D):
    from titan_b200.ops import moe

    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)])
    plan = moe.make_plan(idx, E)
    ref = moe.make_plan(idx.cpu(), E)
    assert torch.equal(plan.dest.cpu(), ref.dest) and torch.equal(plan.offs.cpu(), ref.offs)
    assert torch.equal(plan.counts.cpu(), ref.counts)
    assert all(int(o) % 128 == 0 for o in plan.offs.tolist())
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    gate = torch.rand(T, k, device="cuda", requires_grad=True)
    xp = moe.permute(x, plan, scale=gate)
    xr, gr = x.detach().cpu().float().requires_grad_(), gate.detach().cpu().requires_grad_()
    xp_ref = moe.permute(xr, ref, scale=gr)
    last = int(plan.offs[-1])  # rows beyond are unused capacity and never initialised
    torch.testing.assert_close(xp[:last].float().cpu(), xp_ref[:last], rtol=2e-2, atol=2e-2)
    # padding rows are exactly zero
    used = torch.zeros(plan.capacity, dtype=torch.bool)
    used[ref.dest.long()] = True
    assert torch.all(xp[:last].float().cpu()[~used[:last]] == 0)
    w = torch.rand(T, k, device="cuda", requires_grad=True)
    base = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        xp[last:] = 0  # keeps the comparison of gradients below free of uninitialised values
    out = moe.combine(xp, plan, T, weights=w, base=base)
    wr = w.detach().cpu().requires_grad_()
    out_ref = moe.combine(xp_ref, ref, T, weights=wr, base=base.cpu().float())
    torch.testing.assert_close(out.float().cpu(), out_ref, rtol=3e-2, atol=3e-2)
    g = torch.randn_like(out)
    out.backward(g)
    out_ref.backward(g.float().cpu())
    torch.testing.assert_close(x.grad.float().cpu(), xr.grad, rtol=5e-2, atol=5e-2)
    torch.testing.assert_close(w.grad.cpu(), wr.grad, rtol=5e-2, atol=0.5)
    torch.testing.assert_close(gate.grad.cpu(), gr.grad, rtol=5e-2, atol=0.5)


@pytest.mark.parametrize("G,N,K", [(8, 512, 256), (4, 2816, 2048), (3, 264, 136)])
def test_grouped_linear_fwd_bwd(G, N, K):
    from titan_b200.ops import _lib, moe

    counts = torch.randint(0, 400, (G,))
    counts[1] = 0  # an expert without tokens
    padded = (counts + 127) // 128 * 128
    offs = torch.cumsum(padded, 0).to(torch.int32).cuda()
    cap = int(offs[-1]) + 256  # some unused capacity at the end
    x = torch.zeros(cap, K, device="cuda", dtype=torch.bfloat16)
    start = 0
    for g in range(G):
        x[start:start + int(counts[g])] = torch.randn(int(counts[g]), K, device="cuda")
        start += int(padded[g])
    x.requires_grad_()
    w = (torch.randn(G, N, K, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    if K % 64:
        pytest.skip("dgrad needs K % 64 == 0")
    y = moe.grouped_linear(x, w, offs)
    _lib.shared_status().raise_if_set("grouped gemm")
    last = int(offs[-1])
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = moe.grouped_linear_ref(xr, wr, offs)
    torch.testing.assert_close(y[:last].float(), yr[:last], rtol=2e-2, atol=2e-2)
    g = torch.zeros_like(y)
    g[:last] = torch.randn(last, N, device="cuda")
    g[:last][x.detach()[:last].abs().sum(-1) == 0] = 0  # gradients of padding rows are zero in the real flow
    y.backward(g)
    yr.backward(g.float())
    torch.testing.assert_close(x.grad[:last].float(), xr.grad[:last], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=0.25)
    assert torch.all(w.grad[1] == 0)


def test_fused_moe_matches_baseline():
    from titan_b200.converters.gmm import GMMStateDictUpdater
    from titan_b200.models.deepseek_v3 import deepseekv3_configs
    from titan_b200.protocols import converter as conv

    def build(fused):
        cfg = deepseekv3_configs["smoketest"]()
        cfg.dim, cfg.moe_inter_dim, cfg.inter_dim = 256, 128, 512
        cfg.moe_args.use_grouped_mm = False
        m = cfg.build()
        if fused:
            conv.ModelConvertersContainer([conv.get_model_converter_config(n) for n in
                                           ("b200_moe_dispatch", "b200_gmm")]).convert(m)
        return m

    torch.manual_seed(1)
    base = build(False)
    base.init_states()
    fused = build(True)
    fused.load_state_dict(GMMStateDictUpdater.from_hf({k: v.clone() for k, v in base.state_dict().items()}),
                          strict=False)
    base, fused = base.cuda().bfloat16(), fused.cuda().bfloat16()
    base.init_states(buffer_device="cuda") if False else None
    tokens = torch.randint(0, 2048, (2, 128), device="cuda")
    for m in (base, fused):
        m.freqs_cis = m._precompute("cuda")
    out_b = base(tokens)
    out_f = fused(tokens)
    rel = (out_f.float() - out_b.float()).norm() / out_b.float().norm()
    assert rel < 3e-2, rel
    out_f.float().mean().backward()
    assert all(torch.isfinite(p.grad).all() for p in fused.parameters() if p.grad is not None)
