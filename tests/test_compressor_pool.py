"""Compressor pooling: the PyTorch form against a literal per-block loop (CPU), and the CUDA kernels against the
PyTorch form in fp32 (forward, and the gradients of kv / score / ape)."""

import pytest
import torch

from titan_b200.ops.compressor_pool import compressor_pool, compressor_pool_ref


def _loop(kv, score, ape, r, d, overlap):
    B, S, _ = kv.shape
    out = torch.zeros(B, S // r, d, dtype=kv.dtype)
    for b in range(B):
        for c in range(S // r):
            cands_k, cands_s = [], []
            if overlap and c > 0:
                for i in range(r):
                    t = (c - 1) * r + i
                    cands_k.append(kv[b, t, :d]); cands_s.append(score[b, t, :d] + ape[i, :d])
            for i in range(r):
                t = c * r + i
                lo = d if overlap else 0
                cands_k.append(kv[b, t, lo:lo + d]); cands_s.append(score[b, t, lo:lo + d] + ape[i, lo:lo + d])
            k, s = torch.stack(cands_k), torch.stack(cands_s)
            out[b, c] = (k * s.softmax(0)).sum(0)
    return out


@pytest.mark.parametrize("r,overlap", [(4, True), (8, False)])
def test_reference_matches_loop(r, overlap):
    torch.manual_seed(0)
    B, S, d = 2, 32, 8
    w = 2 * d if overlap else d
    kv, score, ape = torch.randn(B, S, w, dtype=torch.float64), torch.randn(B, S, w, dtype=torch.float64), \
        torch.randn(r, w, dtype=torch.float64)
    torch.testing.assert_close(compressor_pool_ref(kv, score, ape, r, d, overlap), _loop(kv, score, ape, r, d, overlap))


@pytest.mark.gpu
@pytest.mark.parametrize("r,overlap,d", [(4, True, 512), (128, False, 512), (4, True, 128), (128, False, 64)])
def test_kernels_match_reference(r, overlap, d):
    torch.manual_seed(1)
    B, S = 2, 1024
    w = 2 * d if overlap else d
    mk = lambda *s: torch.randn(*s, device="cuda", dtype=torch.float32)
    kv, score, ape = mk(B, S, w), mk(B, S, w) * 2, mk(r, w)
    a = [t.clone().requires_grad_(True) for t in (kv, score, ape)]
    b = [t.clone().requires_grad_(True) for t in (kv, score, ape)]
    out = compressor_pool(*a, r, d, overlap)
    ref = compressor_pool_ref(*b, r, d, overlap)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g)
    for x, y, name in zip(a, b, ("dkv", "dscore", "dape")):
        torch.testing.assert_close(x.grad, y.grad, rtol=1e-3, atol=1e-3, msg=lambda m, n=name: f"{n}: {m}")
