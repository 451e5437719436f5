"""sm_100a elementwise kernels against plain PyTorch fp32 references of the same op."""

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = dict(rtol=1e-2, atol=1e-2)


@pytest.fixture(autouse=True)
def _need_cuda(cuda_device):
    torch.manual_seed(0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,dim", [(37, 256), (512, 4096), (5, 1536), (1000, 128), (333, 512), (129, 1024),
                                      (64, 2048), (77, 8192), (9, 16384), (4099, 4096)])
def test_rmsnorm_fwd_bwd(dtype, rows, dim):
    from titan_b200.ops.norm import rms_norm

    x = torch.randn(rows, dim, device="cuda", dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(dtype).requires_grad_()
    g = torch.randn(rows, dim, device="cuda", dtype=dtype)
    y = rms_norm(x, w, 1e-5)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, **TOL)
    torch.testing.assert_close(x.grad.float(), xr.grad, **TOL)
    # dw sums over rows: tolerance scales with sqrt(rows) in bf16
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=2e-2 * max(1.0, rows ** 0.5 / 4))


def test_rmsnorm_bwd_is_deterministic():
    from titan_b200.ops.norm import rms_norm_bwd, rms_norm_fwd

    x = torch.randn(1000, 4096, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(4096, device="cuda", dtype=torch.bfloat16)
    g = torch.randn_like(x)
    _, rstd = rms_norm_fwd(x, w, 1e-5)
    a = rms_norm_bwd(g, x, w, rstd)
    b = rms_norm_bwd(g, x, w, rstd)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("with_pos", [False, True])
def test_rope_interleaved(dtype, with_pos):
    from titan_b200.models.common import rope as ref
    from titan_b200.ops.rope import rope_apply

    B, S, H, D = 2, 96, 4, 64
    cache = ref.precompute_freqs_cis(D, 256, 500000.0).cuda()
    x = torch.randn(B, S, H, D, device="cuda", dtype=dtype, requires_grad=True)
    pos = torch.randint(0, 256, (B, S), device="cuda") if with_pos else None
    y = rope_apply(x, cache, pos, interleaved=True)
    xr = x.detach().float().requires_grad_()
    yr = ref.apply_rotary_emb_single_complex(xr, cache, pos)
    torch.testing.assert_close(y.float(), yr, **TOL)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    torch.testing.assert_close(x.grad.float(), xr.grad, **TOL)
    # inverse undoes the rotation
    back = rope_apply(y.detach(), cache, pos, interleaved=True, inverse=True)
    torch.testing.assert_close(back.float(), x.detach().float(), rtol=2e-2, atol=2e-2)


def test_rope_half_layout():
    from titan_b200.models.common import rope as ref
    from titan_b200.ops.rope import rope_apply

    B, S, H, D = 2, 64, 8, 128
    cache = ref.precompute_rope_cache(D, 128, 1e6).cuda()
    q = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, S, 2, D, device="cuda", dtype=torch.bfloat16)
    qr, kr = ref.apply_rotary_emb_cos_sin(q.float(), k.float(), cache)
    torch.testing.assert_close(rope_apply(q, cache, interleaved=False).float(), qr, **TOL)
    torch.testing.assert_close(rope_apply(k, cache, interleaved=False).float(), kr, **TOL)


def test_rope_reports_bad_position():
    from titan_b200.models.common import rope as ref
    from titan_b200.ops import _lib
    from titan_b200.ops.rope import rope_apply

    cache = ref.precompute_freqs_cis(64, 32, 1e4).cuda()
    x = torch.randn(1, 8, 2, 64, device="cuda", dtype=torch.bfloat16)
    pos = torch.full((1, 8), 1000, device="cuda")
    rope_apply(x, cache, pos)
    with pytest.raises(_lib.KernelError):
        _lib.shared_status().raise_if_set("rope")


@pytest.mark.parametrize("limit", [0.0, 1.5])
@pytest.mark.parametrize("fused", [False, True])
def test_swiglu(limit, fused):
    from titan_b200.ops.swiglu import swiglu, swiglu_fused, swiglu_ref

    rows, H = 300, 1408
    x = torch.randn(rows, 2 * H, device="cuda", dtype=torch.bfloat16) * 2
    score = torch.rand(rows, device="cuda") if fused else None
    xr = x.detach().float().requires_grad_()
    sr = score.detach().clone().requires_grad_() if fused else None
    ref = swiglu_ref(xr[:, :H], xr[:, H:], sr, limit)
    if fused:
        xi = x.clone().requires_grad_()
        si = score.clone().requires_grad_()
        out = swiglu_fused(xi, si, limit)
    else:
        a = x[:, :H].contiguous().requires_grad_()
        b = x[:, H:].contiguous().requires_grad_()
        out = swiglu(a, b, None, limit)
    torch.testing.assert_close(out.float(), ref, **TOL)
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g.float())
    if fused:
        torch.testing.assert_close(xi.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(si.grad, sr.grad, rtol=2e-2, atol=0.3)
    else:
        torch.testing.assert_close(a.grad.float(), xr.grad[:, :H], rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(b.grad.float(), xr.grad[:, H:], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype,V", [(torch.bfloat16, 2048), (torch.float32, 1000), (torch.bfloat16, 128256)])
def test_cross_entropy(dtype, V):
    from titan_b200.ops.cross_entropy import cross_entropy_ref, cross_entropy_sum

    T = 64
    logits = (torch.randn(T, V, device="cuda") * 3).to(dtype).requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    loss = cross_entropy_sum(logits, labels)
    (loss / 13.0).backward()
    lr = logits.detach().float().requires_grad_()
    ref = cross_entropy_ref(lr, labels)
    (ref / 13.0).backward()
    torch.testing.assert_close(loss, ref, rtol=1e-3, atol=1e-2)
    torch.testing.assert_close(logits.grad.float(), lr.grad, rtol=2e-2, atol=1e-3)


@pytest.mark.parametrize("pdt,gdt", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32)])
def test_fused_adamw_matches_torch(pdt, gdt):
    from titan_b200.optim.fused_adamw import FusedAdamW

    sizes = [(1000,), (257, 33), (4096, 512), (7,)] * 8  # > 24 tensors: exercises launch splitting
    ps = [torch.randn(*s, device="cuda").to(pdt) for s in sizes]
    ref_ps = [p.detach().float().clone().requires_grad_() for p in ps]
    ps = [p.requires_grad_() for p in ps]
    opt = FusedAdamW(ps, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref = torch.optim.AdamW(ref_ps, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(3):
        for p, r in zip(ps, ref_ps):
            g = torch.randn_like(r)
            p.grad = g.to(gdt)
            r.grad = g.to(gdt).float()
        opt.step()
        ref.step()
    for p, r in zip(ps, ref_ps):
        tol = dict(rtol=2e-2, atol=2e-2) if pdt == torch.bfloat16 else dict(rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(p.detach().float(), r.detach(), **tol)
    assert opt.launches > 0


def test_fused_adamw_grad_scale():
    from titan_b200.optim.fused_adamw import FusedAdamW

    p = torch.randn(5000, device="cuda").requires_grad_()
    r = p.detach().clone().requires_grad_()
    g = torch.randn(5000, device="cuda")
    opt = FusedAdamW([p], lr=1e-2, weight_decay=0.0)
    opt.grad_scale = torch.tensor(0.25, device="cuda")
    ref = torch.optim.AdamW([r], lr=1e-2, weight_decay=0.0)
    p.grad, r.grad = g.clone(), g * 0.25
    opt.step()
    ref.step()
    torch.testing.assert_close(p.detach(), r.detach(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("n", [64, 128, 256, 512])
def test_hadamard_matches_matrix_product(n):
    import scipy.linalg

    from titan_b200.ops.hadamard import hadamard, hadamard_ref

    x = torch.randn(3, 37, n, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    H = torch.tensor(scipy.linalg.hadamard(n), dtype=torch.float32, device="cuda")
    y = hadamard(x)
    ref = (x.detach().float() @ H) * n ** -0.5
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(hadamard_ref(x.detach(), n ** -0.5).float(), ref, rtol=2e-2, atol=2e-2)
    g = torch.randn_like(y)
    y.backward(g)
    torch.testing.assert_close(x.grad.float(), (g.float() @ H) * n ** -0.5, rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_multi_tensor_sum_of_squares(dtype):
    from titan_b200.ops.multi_tensor import sum_of_squares

    torch.manual_seed(0)
    # sizes around the 65536-element chunk, a ragged tail, a tensor spanning several launches, an unaligned view
    big = torch.randn(70_000_000, device="cuda").to(dtype)
    ts = [torch.randn(n, device="cuda").to(dtype) for n in (1, 7, 65535, 65536, 65537, 1_000_003)] + [big]
    ts.append(torch.randn(4099, device="cuda").to(dtype)[3:])
    got = sum_of_squares(ts)
    ref = sum(t.double().pow(2).sum() for t in ts)
    assert abs(float(got) - float(ref)) / float(ref) < 1e-4
