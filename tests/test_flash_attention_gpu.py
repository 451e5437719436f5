"""tcgen05 flash-attention forward and backward against fp32 PyTorch attention: causal, GQA, packed documents."""

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
    out = _FlashFn.apply(q, k, v, scale, None)
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


def _ref_docs(q, k, v, scale, seq_start):
    """fp32 attention with the causal + same-document mask built from `seq_start` [B, S]."""
    B, H, S, D = q.shape
    rep = H // k.shape[1]
    kf, vf = k.float().repeat_interleave(rep, 1), v.float().repeat_interleave(rep, 1)
    s = (q.float() @ kf.transpose(-1, -2)) * scale
    pos = torch.arange(S, device=q.device)
    allowed = (pos[None, :] <= pos[:, None])[None] & (pos[None, None, :] >= seq_start[:, :, None].long())   # [B, S, S]
    s = s.masked_fill(~allowed[:, None], float("-inf"))
    return torch.softmax(s, -1) @ vf


@pytest.mark.parametrize("B,S,H,Hkv", [(1, 256, 4, 2), (2, 512, 4, 4), (1, 1024, 8, 2)])
def test_flash_backward_kernel_matches_fp32_autograd(B, S, H, Hkv):
    from titan_b200.ops import _lib
    from titan_b200.ops.flash_attention import flash_attention

    mk = lambda h: (torch.randn(B, S, h, 128, device="cuda") * 0.7).to(torch.bfloat16).transpose(1, 2)  # noqa: E731
    q, k, v = mk(H), mk(Hkv), mk(Hkv)
    g = torch.randn(B, S, H, 128, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
    ql, kl, vl = (t.detach().clone().requires_grad_() for t in (q, k, v))
    before = _lib.launch_count()
    flash_attention(ql, kl, vl).backward(g)
    _lib.shared_status().raise_if_set("flash_attention")
    assert _lib.launch_count() == before + 2          # one forward, one backward kernel
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref, _ = _ref(qr, kr, vr, 128 ** -0.5)
    ref.backward(g.float())
    for a, b_, name in zip((ql, kl, vl), (qr, kr, vr), ("dq", "dk", "dv")):
        torch.testing.assert_close(a.grad.float(), b_.grad, rtol=3e-2, atol=3e-2, msg=lambda m, n=name: f"{n}: {m}")


@pytest.mark.parametrize("bounds", [[[0, 100, 128, 300, 512]], [[0, 512]], [[0, 7, 260, 511, 512], [0, 384, 512]]])
def test_packed_documents_forward_and_backward(bounds):
    """Documents of a packed sequence attend only to themselves: boundaries inside a block, on a block edge, a
    document spanning several blocks, and one-token documents."""
    from titan_b200.models.common.varlen_attention import VarlenAttention, VarlenMetadata
    from titan_b200.ops import _lib

    B, S, H, Hkv = len(bounds), 512, 4, 2
    meta = VarlenMetadata(bounds, max(e - a for row in bounds for a, e in zip(row[:-1], row[1:])))
    mk = lambda h: (torch.randn(B, S, h, 128, device="cuda") * 0.7).to(torch.bfloat16).transpose(1, 2)  # noqa: E731
    q, k, v = mk(H), mk(Hkv), mk(Hkv)
    g = torch.randn(B, S, H, 128, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
    ql, kl, vl = (t.detach().clone().requires_grad_() for t in (q, k, v))
    before = _lib.launch_count()
    out = VarlenAttention()(ql, kl, vl, scale=128 ** -0.5, attn_mask=meta)
    out.backward(g)
    _lib.shared_status().raise_if_set("flash_attention")
    assert _lib.launch_count() == before + 2          # the whole packed batch: one forward, one backward launch
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _ref_docs(qr, kr, vr, 128 ** -0.5, meta.seq_start("cuda"))
    ref.backward(g.float())
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    for a, b_, name in zip((ql, kl, vl), (qr, kr, vr), ("dq", "dk", "dv")):
        torch.testing.assert_close(a.grad.float(), b_.grad, rtol=3e-2, atol=3e-2, msg=lambda m, n=name: f"{n}: {m}")
