"""Block-scaled MXFP8 GEMM: scale-atom packing (CPU) and the tcgen05 kernel against the fp32 dequantise-and-multiply
reference (GPU)."""

import pytest
import torch

from titan_b200.ops.mxfp8_gemm import mxfp8_gemm, mxfp8_gemm_ref, pack_scale_atoms


def test_scale_atoms_layout():
    R, KB = 200, 8  # 200 rows -> 2 row blocks (padded with 1.0 = 127); 8 K-blocks -> 2 stages
    s = (torch.arange(R * KB) % 251).to(torch.uint8).view(R, KB)
    atoms = pack_scale_atoms(s)
    assert atoms.shape == (2, 2, 512)
    for row, blk in [(0, 0), (5, 3), (37, 1), (127, 7), (128, 4), (199, 6)]:
        rb, m1, m0 = row // 128, (row % 128) // 32, row % 32
        assert atoms[rb, blk // 4, m0 * 16 + m1 * 4 + blk % 4] == s[row, blk]
    assert atoms[1, 0, (210 % 32) * 16 + ((210 % 128) // 32) * 4] == 127  # padded row


@pytest.mark.gpu
@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 384, 512), (1024, 1032, 1024)])
def test_kernel_matches_dequantised_reference(M, N, K, tile_n):
    from titan_b200.lowp.mx import mx_quantize
    from titan_b200.ops import _lib

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16) * torch.logspace(-2, 2, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    aq, sa = mx_quantize(a, -1)
    bq, sb = mx_quantize(b, -1)
    out = mxfp8_gemm(aq, sa, bq, sb, tile_n=tile_n)
    ref = mxfp8_gemm_ref(aq, sa, bq, sb)
    torch.cuda.synchronize()
    _lib.shared_status().raise_if_set("mxfp8 gemm")
    err = (out.float() - ref).abs().max() / ref.abs().max()
    assert err < 8e-3, err  # bf16 output rounding only: the operands are exact


@pytest.mark.gpu
@pytest.mark.parametrize("tile_n", [0, 128])
def test_grouped_modes_match_per_expert_products(tile_n, cuda_device):
    """Forward (expert picks its weight rows), input gradient (expert picks a contraction slice of the transposed
    weight) and weight gradient (contraction over the expert's rows), with an expert without rows and padding rows
    after the last group."""
    from titan_b200.lowp.mx import mx_dequantize_ref, mx_quantize_dual
    from titan_b200.ops.mxfp8_gemm import GROUP_B_ROWS, GROUP_B_SLICE, GROUP_K, mxfp8_grouped_gemm

    torch.manual_seed(11)
    E, N, K = 4, 384, 256
    sizes = [256, 0, 128, 384]
    T = sum(sizes) + 128  # one tile of padding rows at the end
    offs = torch.tensor(sizes, device="cuda").cumsum(0).to(torch.int32)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(E, N, K, device="cuda", dtype=torch.bfloat16) * 0.1)
    g = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
    xq1, xs1, xq2t, xs2t = mx_quantize_dual(x)
    wq1, ws1, wq2t, ws2t = mx_quantize_dual(w.reshape(E * N, K))
    gq1, gs1, gq2t, gs2t = mx_quantize_dual(g)
    deq = lambda q, s: mx_dequantize_ref(q, s, -1, torch.float32)  # noqa: E731
    xd, wd, gd = deq(xq1, xs1), deq(wq1, ws1).view(E, N, K), deq(gq1, gs1)
    wtd = deq(wq2t, ws2t).view(K, E, N)       # weight blocked down its N rows, transposed
    gtd, xtd = deq(gq2t, gs2t), deq(xq2t, xs2t)  # [N, T], [K, T]

    y = mxfp8_grouped_gemm(xq1, xs1, wq1, ws1, offs, GROUP_B_ROWS, tile_n=tile_n).float()
    dx = mxfp8_grouped_gemm(gq1, gs1, wq2t, ws2t, offs, GROUP_B_SLICE, tile_n=tile_n).float()
    dw = mxfp8_grouped_gemm(gq2t, gs2t, xq2t, xs2t, offs, GROUP_K, tile_n=tile_n).float().view(E, N, K)
    torch.cuda.synchronize()
    start = 0
    for e, end in enumerate(offs.tolist()):
        if end > start:
            ref_y = xd[start:end] @ wd[e].t()
            ref_dx = gd[start:end] @ wtd[:, e].t()
            ref_dw = gtd[:, start:end] @ xtd[:, start:end].t()
            for got, ref in ((y[start:end], ref_y), (dx[start:end], ref_dx), (dw[e], ref_dw)):
                assert torch.allclose(got, ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item())
                assert (got - ref).pow(2).sum() < 1e-4 * ref.pow(2).sum()
        else:
            assert dw[e].abs().max() == 0  # an expert without rows gets a zero gradient, not stale memory
        start = end
    assert y[start:].abs().max() == 0 and dx[start:].abs().max() == 0  # padding rows are written as zeros


@pytest.mark.gpu
def test_aligned_grouped_mm_autograd_matches_the_loop_over_experts(cuda_device):
    from titan_b200.lowp.mx_linear import mx_grouped_mm
    from titan_b200.ops import _lib

    torch.manual_seed(12)
    E, N, K = 3, 256, 128
    sizes = [128, 256, 0]
    offs = torch.tensor(sizes, device="cuda").cumsum(0).to(torch.int32)
    T = sum(sizes) + 127 * E  # the capacity bound of the padded layout: not a multiple of 128
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    x[sum(sizes):] = float("nan")  # unused capacity holds anything
    x.requires_grad_()
    w = (torch.randn(E, N, K, device="cuda", dtype=torch.bfloat16) * 0.1).requires_grad_()
    g = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
    g[sum(sizes):] = float("nan")
    before = _lib.launch_count()
    y = mx_grouped_mm(x, w, offs, aligned=True)
    y.backward(g)
    assert _lib.launch_count() - before == 7  # 4 quantiser passes + 3 grouped GEMMs, whatever the number of experts
    got = (y.detach().float(), x.grad.float(), w.grad.float())
    n = sum(sizes)
    assert y.shape == (T, N) and all(t[n:].abs().max() == 0 for t in got[:2])  # unused rows: zeros, never NaN
    x.grad = w.grad = None
    y2 = mx_grouped_mm(x, w, offs)
    y2.backward(g)
    for a, b in zip(got, (y2.detach().float()[:n], x.grad.float()[:n], w.grad.float())):
        a = a[:n] if a.shape[0] == T else a
        assert torch.isfinite(a).all() and (a - b).pow(2).sum() <= 1e-4 * b.pow(2).sum()


@pytest.mark.gpu
def test_expert_weight_quantisation_is_kept_between_optimizer_steps(cuda_device):
    """With a `weight_key` the grouped MX product quantises the weight once (both views from one dual-axis pass) and
    reuses it in forward, recomputed forward and input gradient; an invalidation or an in-place update refreshes it."""
    from titan_b200.lowp import mx_linear
    from titan_b200.ops import _lib

    torch.manual_seed(3)
    E, N, K, rows = 2, 256, 256, 256
    offs = torch.tensor([rows, 2 * rows], device="cuda", dtype=torch.int32)
    x = torch.randn(2 * rows, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(E, N, K, device="cuda", dtype=torch.bfloat16) * 0.1).requires_grad_()
    g = torch.randn(2 * rows, N, device="cuda", dtype=torch.bfloat16)

    def run(key):
        x.grad = w.grad = None
        before = _lib.launch_count()
        y = mx_linear.mx_grouped_mm(x, w, offs, aligned=True, weight_key=key)
        y.backward(g)
        return y.detach().clone(), x.grad.clone(), w.grad.clone(), _lib.launch_count() - before

    mx_linear.invalidate_weight_cache()
    plain = run(None)
    first = run("w")      # fills the cache: one weight pass instead of two
    second = run("w")     # reuses it: no weight pass at all
    for a, b in zip(plain[:3], first[:3]):
        assert torch.equal(a, b)
    for a, b in zip(first[:3], second[:3]):
        assert torch.equal(a, b)
    assert first[3] == plain[3] - 1 and second[3] == plain[3] - 2
    with torch.no_grad():
        w.mul_(2.0)       # in-place update: the version counter moves, the views are rebuilt
    third = run("w")
    assert third[3] == first[3]
    torch.testing.assert_close(third[0].float(), 2 * first[0].float(), rtol=2e-2, atol=2e-2)
    # a raw-pointer update (what the fused optimizer kernels do) is invisible to the counter: the trainer invalidates
    w.data = w.data * 0.5
    mx_linear.invalidate_weight_cache()
    fourth = run("w")
    torch.testing.assert_close(fourth[0].float(), first[0].float(), rtol=2e-2, atol=2e-2)
