"""Hyper-connection kernels against the fp32 PyTorch statement of the same math (forward and all gradients)."""

import pytest
import torch

from titan_b200.ops import mhc

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_cuda(cuda_device):
    torch.manual_seed(0)


def _params(D, dev):
    fn = (torch.randn(24, 4 * D, device=dev) * 0.05).requires_grad_()
    scale = (torch.randn(3, device=dev) * 0.5 + 1.0).requires_grad_()
    base = (torch.randn(24, device=dev) * 0.3).requires_grad_()
    return fn, scale, base


@pytest.mark.parametrize("T,D", [(37, 256), (64, 1024), (16, 4096), (5, 7168)])
def test_mhc_pre_matches_reference(T, D):
    from titan_b200.ops.mhc_cuda import mhc_pre

    dev = "cuda"
    x = torch.randn(T, 4, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    fn, scale, base = _params(D, dev)
    y, post, comb = mhc_pre(x, fn, scale, base, 20, 1e-6, 1e-6)
    xr = x.detach().float().requires_grad_()
    fnr, sr, br = (t.detach().clone().requires_grad_() for t in (fn, scale, base))
    yr, postr, combr = mhc.hc_pre_ref(xr, fnr, sr, br, 4, 20, 1e-6, 1e-6)
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(post, postr, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(comb, combr, rtol=2e-3, atol=2e-3)
    gy = torch.randn_like(yr)
    gp, gc = torch.randn_like(postr), torch.randn_like(combr)
    (y.float() * gy).sum().add((post * gp).sum()).add((comb * gc).sum()).backward()
    (yr * gy).sum().add((postr * gp).sum()).add((combr * gc).sum()).backward()
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=5e-2, atol=5e-2)

    def rel(a, b):
        return (a.float() - b).norm() / b.norm().clamp_min(1e-6)

    assert rel(fn.grad, fnr.grad) < 3e-2, rel(fn.grad, fnr.grad)
    assert rel(scale.grad, sr.grad) < 3e-2, (scale.grad, sr.grad)
    assert rel(base.grad, br.grad) < 3e-2, (base.grad, br.grad)


@pytest.mark.parametrize("T,D", [(37, 256), (16, 4096)])
def test_hc_head_runs_the_fused_pre_kernel_and_matches_reference(T, D):
    from titan_b200.ops import _lib

    dev = "cuda"
    x = torch.randn(T, 4, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    fn = (torch.randn(4, 4 * D, device=dev) * 0.05).requires_grad_()
    scale = (torch.randn(1, device=dev) * 0.5 + 1.0).requires_grad_()
    base = (torch.randn(4, device=dev) * 0.3).requires_grad_()
    mhc.set_fused(pre=True)
    try:
        before = _lib.launch_count()
        y = mhc.hc_head(x, fn, scale, base)
        assert _lib.launch_count() > before
    finally:
        mhc.set_fused(pre=False)
    xr = x.detach().float().requires_grad_()
    fnr, sr, br = (t.detach().clone().requires_grad_() for t in (fn, scale, base))
    yr = mhc.hc_head_ref(xr, fnr, sr, br)
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    gy = torch.randn_like(yr)
    (y.float() * gy).sum().backward()
    (yr * gy).sum().backward()
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=5e-2, atol=5e-2)

    def rel(a, b):
        return (a.float() - b).norm() / b.norm().clamp_min(1e-6)

    assert rel(fn.grad, fnr.grad) < 3e-2 and rel(scale.grad, sr.grad) < 3e-2 and rel(base.grad, br.grad) < 3e-2


@pytest.mark.parametrize("T,D", [(33, 256), (16, 4096), (3, 7168)])
def test_mhc_post_matches_reference(T, D):
    from titan_b200.ops.mhc_cuda import mhc_post

    dev = "cuda"
    y = torch.randn(T, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    res = torch.randn(T, 4, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    post = torch.rand(T, 4, device=dev, requires_grad=True)
    comb = torch.rand(T, 4, 4, device=dev, requires_grad=True)
    out = mhc_post(y, res, post, comb)
    yr, rr, pr, cr = (t.detach().float().requires_grad_() for t in (y, res, post, comb))
    outr = mhc.hc_post_ref(yr, rr, pr, cr)
    torch.testing.assert_close(out.float(), outr, rtol=2e-2, atol=2e-2)
    g = torch.randn_like(outr)
    out.backward(g.to(out.dtype))
    outr.backward(g.to(torch.bfloat16).float())
    torch.testing.assert_close(y.grad.float(), yr.grad, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(res.grad.float(), rr.grad, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(post.grad, pr.grad, rtol=3e-2, atol=3e-1)
    torch.testing.assert_close(comb.grad, cr.grad, rtol=3e-2, atol=3e-1)


def test_converters_switch_the_dispatch_and_model_still_matches():
    from titan_b200.models.deepseek_v4 import DeepSeekV4Model, deepseekv4_configs

    cfg = deepseekv4_configs["smoketest"]()
    cfg.max_seq_len = 128
    with torch.device("cuda"):
        model = DeepSeekV4Model(cfg)
    model.init_states(buffer_device=torch.device("cuda"))
    model.bfloat16()
    tok = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda")
    ref = model(tok).float()
    mhc.set_fused(pre=True, post=True)
    try:
        before = __import__("titan_b200.ops._lib", fromlist=["x"]).launch_count()
        out = model(tok).float()
        out.logsumexp(-1).mean().backward()
        assert __import__("titan_b200.ops._lib", fromlist=["x"]).launch_count() > before
    finally:
        mhc.set_fused(pre=False, post=False)
    assert (out - ref).abs().max() < 0.15, (out - ref).abs().max()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
