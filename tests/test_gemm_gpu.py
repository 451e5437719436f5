"""tcgen05 GEMM against a PyTorch fp32 reference, all operand storage combinations."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_cuda(cuda_device):
    torch.manual_seed(0)


def _check(M, N, K, a_mn, b_mn, dtype=torch.bfloat16, out_dtype=None, max_ctas=0):
    from titan_b200.ops import _lib
    from titan_b200.ops.gemm import gemm, gemm_ref

    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=dtype)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=dtype)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=out_dtype, max_ctas=max_ctas)
    _lib.shared_status().raise_if_set("gemm")
    ref = gemm_ref(a, b, a_mn, b_mn, out_dtype=torch.float32)
    # bf16 inputs are exact in fp32 products; error comes from the output rounding and summation order
    scale = K ** 0.5
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2 * scale)
    rel = (out.float() - ref).norm() / ref.norm()
    assert rel < 5e-3, f"relative error {rel}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 512), (384, 768, 1024)])
def test_gemm_kmajor_exact_tiles(M, N, K):
    _check(M, N, K, False, False)


@pytest.mark.parametrize("M,N,K", [(100, 200, 72), (130, 264, 200), (1, 8, 8), (2049, 1032, 520)])
def test_gemm_kmajor_ragged(M, N, K):
    _check(M, N, K, False, False)


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (200, 328, 136)])
def test_gemm_mn_major(a_mn, b_mn, M, N, K):
    _check(M, N, K, a_mn, b_mn)


def test_gemm_fp16_and_fp32_out():
    _check(256, 256, 256, False, False, dtype=torch.float16)
    _check(256, 256, 256, False, False, out_dtype=torch.float32)


def test_gemm_many_tiles_per_cta():
    # few CTAs → each walks several tiles: exercises accumulator double-buffering and phase flips
    _check(1024, 1024, 320, False, False, max_ctas=3)


def test_gemm_accumulate():
    from titan_b200.ops.gemm import gemm

    a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    out = torch.ones(256, 256, device="cuda", dtype=torch.float32)
    gemm(a, b, out=out, accumulate=True)
    ref = 1 + a.float() @ b.float().t()
    torch.testing.assert_close(out, ref, rtol=1e-3, atol=1e-2)


def test_linear_autograd_matches_torch():
    from titan_b200.ops.gemm import linear

    x = torch.randn(4, 96, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(768, 512, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    y = linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=5e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=0.3)
