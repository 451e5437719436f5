"""tcgen05 flash-attention forward against fp32 PyTorch attention (causal, GQA), and the op's autograd path."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_cuda(cuda_device):
    torch.manual_seed(0)


def _ref(q, k, v, scale):
    B, H, S, D = q.shape
    rep = H // k.shape[1]
    kf, vf = k.float().repeat_interleave(rep, 1), v.float().repeat_interleave(rep, 1)
    s = (q.float() @ kf.transpose(-1, -2)) * scale
    s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    return torch.softmax(s, -1) @ vf, torch.logsumexp(s, -1)


@pytest.mark.parametrize("B,S,H,Hkv", [(1, 128, 2, 2), (2, 384, 4, 2), (1, 1024, 8, 2)])
def test_flash_forward_matches_reference(B, S, H, Hkv):
    from titan_b200.ops import _lib
    from titan_b200.ops.flash_attention import _FlashFn

    q = torch.randn(B, S, H, 128, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
    k = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
    v = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
    scale = 128 ** -0.5
    before = _lib.launch_count()
    out = _FlashFn.apply(q, k, v, scale)
    assert _lib.launch_count() == before + 1
    ref, _ = _ref(q, k, v, scale)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)


def test_flash_op_gradients_match_library():
    from titan_b200.ops.flash_attention import flash_attention

    q, k, v = (torch.randn(1, n, 256, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True) for n in (4, 2, 2))
    g = torch.randn(1, 4, 256, 128, device="cuda", dtype=torch.bfloat16)
    flash_attention(q, k, v).backward(g)
    got = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True).backward(g)
    for a, t in zip(got, (q, k, v)):
        torch.testing.assert_close(a.float(), t.grad.float(), rtol=2e-2, atol=2e-2)
