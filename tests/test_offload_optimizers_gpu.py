"""Swap and Virtual optimizers on a GPU against the resident fused AdamW: bit-identical parameters after three
steps (all three run the same multi-tensor kernel; only where the moments live differs), moments actually off the
device, and peak device memory of the swap pipeline as its docstring states (two slots of two or three moments)."""

import copy

import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu


def _model(device):
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(512, 1024, bias=False), nn.LayerNorm(1024), nn.Linear(1024, 1024),
                         nn.Linear(1024, 256, bias=False)).to(device=device, dtype=torch.bfloat16)


def _steps(model, opt, n=3):
    g = torch.Generator(device="cuda").manual_seed(1)
    for _ in range(n):
        opt.zero_grad()
        x = torch.randn(64, 512, device="cuda", dtype=torch.bfloat16, generator=g)
        model(x).float().pow(2).mean().backward()
        opt.step()
    torch.cuda.synchronize()


@pytest.mark.parametrize("amsgrad", [False, True])
def test_swap_adamw_is_bit_identical_to_resident_fused_adamw(cuda_device, amsgrad):
    from titan_b200.optim.fused_adamw import FusedAdamW
    from titan_b200.optim.swap_optimizer import SwapAdamW

    ref_model = _model(cuda_device)
    model = copy.deepcopy(ref_model)
    kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, amsgrad=amsgrad)
    ref = FusedAdamW(list(ref_model.parameters()), **kw)
    opt = SwapAdamW(list(model.parameters()), swap_times=4, **kw)
    assert len(opt.slices) >= 3 and opt.m_host.is_pinned() and not opt.m_host.is_cuda
    _steps(ref_model, ref)
    before = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    _steps(model, opt)
    opt.synchronize()
    for a, b in zip(ref_model.parameters(), model.parameters()):
        assert torch.equal(a, b)
    # the moments on the host equal the resident ones
    p0, q0 = next(iter(ref_model.parameters())), next(iter(model.parameters()))
    assert torch.equal(ref.state[p0]["exp_avg"].cpu().float().reshape(-1),
                       opt.host_views(q0)["exp_avg"].reshape(-1))
    # staging: 2 slots x (2 or 3) moments x slot_numel fp32, nothing else stays on the device
    n_buf = 2 * (3 if amsgrad else 2)
    staging = n_buf * opt.slot_numel * 4
    grads = sum(p.grad.numel() * p.grad.element_size() for p in model.parameters())
    held = torch.cuda.memory_allocated() - before - grads
    assert held <= staging + n_buf * (2 << 20), (held, staging)   # the caching allocator rounds each buffer up to 2 MiB
    with_staging = torch.cuda.memory_allocated()
    opt.release_staging()
    assert with_staging - torch.cuda.memory_allocated() >= staging   # the moments' only device copies are gone


def test_virtual_adamw_with_a_budget_smaller_than_the_model(cuda_device):
    from titan_b200.optim.fused_adamw import FusedAdamW
    from titan_b200.optim.virtual_optimizer import VirtualAdamW, VirtualAllocator

    ref_model = _model(cuda_device)
    model = copy.deepcopy(ref_model)
    kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref = FusedAdamW(list(ref_model.parameters()), **kw)
    # 6 MB: both moments of the first matrix (2 x 2 MiB) and of the norm fit, the second matrix (params[3], 2 x 4 MiB)
    # does not
    alloc = VirtualAllocator(6e-3)
    opt = VirtualAdamW(list(model.parameters()), allocator=alloc, **kw)
    _steps(ref_model, ref)
    _steps(model, opt)
    for a, b in zip(ref_model.parameters(), model.parameters()):
        assert torch.equal(a, b)
    params = list(model.parameters())
    assert id(params[0]) in opt.virtual_params and id(params[3]) not in opt.virtual_params
    m0 = opt.state[params[0]]["exp_avg"]
    assert not m0.is_cuda and m0.is_pinned()            # read and written in place over the host link
    assert opt.state[params[3]]["exp_avg"].is_cuda      # beyond the budget: ordinary device state
    assert torch.equal(m0.float(), ref.state[next(iter(ref_model.parameters()))]["exp_avg"].cpu().float())


def test_graphed_fused_adamw_matches_the_eager_step(cuda_device):
    """The fused AdamW step replayed from a CUDA graph: bit-identical parameters to the eager launches over steps with a
    changing learning rate and a clip coefficient, re-recorded when a gradient moves to another address."""
    from titan_b200.optim.fused_adamw import FusedAdamW

    ref_model = _model(cuda_device)
    model = copy.deepcopy(ref_model)
    kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref = FusedAdamW(list(ref_model.parameters()), **kw)
    opt = FusedAdamW(list(model.parameters()), cuda_graph=True, **kw)
    g = torch.Generator(device="cuda").manual_seed(1)
    hold = []
    for step in range(6):
        for o in (ref, opt):
            for grp in o.param_groups:
                grp["lr"] = 1e-2 * (1.0 - 0.1 * step)
        scale = torch.tensor(0.5 + 0.1 * step, device="cuda")
        ref.grad_scale, opt.grad_scale = scale, scale.clone()
        x = torch.randn(64, 512, device="cuda", dtype=torch.bfloat16, generator=g)
        for m, o in ((ref_model, ref), (model, opt)):
            o.zero_grad()
            m(x).float().pow(2).mean().backward()
        if step == 3:
            hold = [p.grad for p in model.parameters()]          # keep these alive: the next gradients land elsewhere
        ref.step()
        opt.step()
    torch.cuda.synchronize()
    for a, b in zip(ref_model.parameters(), model.parameters()):
        assert torch.equal(a, b)
    assert opt.graph_replays == 6 and 1 <= opt.graph_captures <= 5, (opt.graph_captures, opt.graph_replays)
    del hold


@pytest.mark.parametrize("shape", [(512, 1024), (1024, 512), (2, 256, 768)])
def test_newton_schulz_on_tensor_cores_matches_the_batched_library_form(cuda_device, shape):
    """Muon's Newton-Schulz iteration with its three products per step on the tcgen05 GEMM against the same iteration
    on batched library products: same bf16 inputs, fp32 accumulation in both."""
    from titan_b200.ops import _lib
    from titan_b200.optim import muon

    torch.manual_seed(0)
    g = torch.randn(*shape, device="cuda", dtype=torch.bfloat16)
    before = _lib.launch_count()
    got = muon.zeropower_via_newtonschulz5(g, steps=5)
    assert _lib.launch_count() - before >= 15          # 3 products x 5 steps (x batch)
    saved = muon.TC_MIN_DIM
    muon.TC_MIN_DIM = 1 << 30
    try:
        ref = muon.zeropower_via_newtonschulz5(g, steps=5)
    finally:
        muon.TC_MIN_DIM = saved
    torch.testing.assert_close(got.float(), ref.float(), rtol=3e-2, atol=3e-2)
    u = got.float() if got.dim() == 2 else got[0].float()
    small, big = sorted(u.shape)
    gram = u @ u.t() if u.shape[0] <= u.shape[1] else u.t() @ u
    assert (gram.diagonal().mean() - 1).abs() < 0.3     # singular values pulled towards 1
