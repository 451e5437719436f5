"""Sparse MLA kernel (gathered key tiles on tcgen05) against the fp32 gather oracle: output, log-sum-exp, teacher,
empty slots, sink logits, head groups, and gradients through the chunked backward."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(S, H, T, K, dq=576, dv=512, empty=0.1, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = (torch.randn(S, H, dq, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    kv = (torch.randn(T, dq, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(T, device="cuda", generator=g)[:K] for _ in range(S)]).to(torch.int32)
    if empty:
        idx = torch.where(torch.rand(S, K, device="cuda", generator=g) < empty, torch.full_like(idx, -1), idx)
    return q, kv, idx


@pytest.mark.parametrize("S,H,T,K,dq,dv", [(8, 16, 512, 128, 576, 512), (40, 16, 4096, 256, 576, 512),
                                           (16, 32, 1024, 384, 576, 512), (8, 64, 1024, 128, 576, 512),
                                           (12, 16, 700, 256, 192, 128)])
def test_forward_matches_gather_oracle(cuda_device, S, H, T, K, dq, dv):
    from titan_b200.ops import _lib
    from titan_b200.ops.sparse_mla import sparse_mla_forward, sparse_mla_forward_ref, sparse_mla_supported

    q, kv, idx = _case(S, H, T, K, dq, dv)
    assert sparse_mla_supported(q, kv, idx, dv)
    scale = dq ** -0.5
    out, lse, teacher = sparse_mla_forward(q, kv, idx, scale, dv)
    _lib.shared_status().raise_if_set("sparse_mla")
    ro, rl, rt = sparse_mla_forward_ref(q, kv, idx, scale, dv)
    torch.testing.assert_close(lse, rl, rtol=1e-3, atol=2e-3)
    torch.testing.assert_close(out.float(), ro.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(teacher, rt, rtol=2e-2, atol=2e-3)


def test_sink_and_fully_empty_rows(cuda_device):
    from titan_b200.ops.sparse_mla import sparse_mla_forward, sparse_mla_forward_ref

    q, kv, idx = _case(8, 16, 512, 128)
    idx[3] = -1                                   # a query without any key
    sink = torch.randn(16, device="cuda")
    scale = 576 ** -0.5
    out, lse, teacher = sparse_mla_forward(q, kv, idx, scale, 512, sink=sink)
    ro, rl, rt = sparse_mla_forward_ref(q, kv, idx, scale, 512, sink=sink)
    torch.testing.assert_close(lse, rl, rtol=1e-3, atol=2e-3)
    torch.testing.assert_close(out.float(), ro.float(), rtol=2e-2, atol=2e-2)
    assert float(out[3].abs().max()) == 0.0       # only the sink holds mass there
    out2, lse2, _ = sparse_mla_forward(q, kv, idx, scale, 512)
    assert torch.isinf(lse2[3]).all() and float(out2[3].abs().max()) == 0.0


@pytest.mark.parametrize("kernel_backward", [True, False])
@pytest.mark.parametrize("S,H,T,K,dq,dv,sink", [(24, 16, 512, 128, 576, 512, False), (20, 32, 900, 256, 576, 512, True),
                                                (9, 64, 640, 384, 192, 128, False), (16, 16, 300, 128, 512, 512, True)])
def test_backward_matches_autograd_of_the_oracle(cuda_device, kernel_backward, S, H, T, K, dq, dv, sink):
    """Both backwards (tensor-core kernel with vector reductions into the latent's rows; chunked PyTorch) against
    autograd through the fp32 oracle: queries, latent (keys + values share rows), sink logits."""
    from titan_b200.ops import _lib, sparse_mla as mod

    q, kv, idx = _case(S, H, T, K, dq, dv, empty=0.2)
    scale = dq ** -0.5
    sk = torch.randn(H, device="cuda") if sink else None
    q1, kv1 = q.clone().requires_grad_(), kv.clone().requires_grad_()
    sk1 = sk.clone().requires_grad_() if sink else None
    saved = mod.KERNEL_BACKWARD
    mod.KERNEL_BACKWARD = kernel_backward
    try:
        out, teacher, lse = mod.sparse_mla(q1, kv1, idx, scale, dv, sk1, chunk=16)
        g = torch.randn_like(out)
        out.backward(g)
        _lib.shared_status().raise_if_set("sparse_mla_bwd")
    finally:
        mod.KERNEL_BACKWARD = saved
    qr, kr = q.float().requires_grad_(), kv.float().requires_grad_()
    skr = sk.clone().requires_grad_() if sink else None
    ro, _, _ = mod.sparse_mla_forward_ref(qr, kr, idx, scale, dv, skr)
    ro.backward(g.float())
    torch.testing.assert_close(q1.grad.float(), qr.grad, rtol=5e-2, atol=2e-2)
    torch.testing.assert_close(kv1.grad.float(), kr.grad, rtol=5e-2, atol=3e-2)
    if sink:
        torch.testing.assert_close(sk1.grad, skr.grad, rtol=5e-2, atol=2e-2)


@pytest.mark.parametrize("S,H,T,K,dq,dv,sink", [(40, 16, 4096, 2048, 576, 512, False), (24, 32, 2000, 1024, 576, 512, True),
                                                (16, 16, 900, 384, 512, 512, True), (9, 16, 600, 256, 320, 256, False)])
def test_pipelined_forward_matches_the_single_tile_kernel(cuda_device, S, H, T, K, dq, dv, sink):
    """The half-tile ring (two buffers of chunks, copies travelling under the tensor-core and softmax work) against
    the single-tile kernel: same output, log-sum-exp and teacher distribution, and both against the fp32 oracle."""
    from titan_b200.ops import _lib, sparse_mla as mod

    q, kv, idx = _case(S, H, T, K, dq, dv, empty=0.15)
    sk = torch.randn(H, device="cuda") if sink else None
    scale = dq ** -0.5
    try:
        mod.set_pipelined(True)
        o1, l1, t1 = mod.sparse_mla_forward(q, kv, idx, scale, dv, sk)
        mod.set_pipelined(False)
        o0, l0, t0 = mod.sparse_mla_forward(q, kv, idx, scale, dv, sk)
    finally:
        mod.set_pipelined(False)
    _lib.shared_status().raise_if_set("sparse_mla")
    torch.testing.assert_close(l1, l0, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(o1.float(), o0.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(t1, t0, rtol=1e-3, atol=1e-4)
    ro, rl, rt = mod.sparse_mla_forward_ref(q, kv, idx, scale, dv, sk)
    torch.testing.assert_close(l1, rl, rtol=1e-3, atol=2e-3)
    torch.testing.assert_close(o1.float(), ro.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(t1, rt, rtol=2e-2, atol=2e-3)
