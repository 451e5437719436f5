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
