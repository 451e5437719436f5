"""DSA: fused path against the eager oracle (CPU), kernels against PyTorch references (GPU)."""

import pytest
import torch


def _inputs(B=1, H=4, S=48, Dq=40, Dv=24, Hi=4, Di=32, device="cpu", dtype=torch.float32):
    torch.manual_seed(0)
    q = torch.randn(B, H, S, Dq, device=device, dtype=dtype, requires_grad=True)
    k = torch.randn(B, 1, S, Dq, device=device, dtype=dtype, requires_grad=True)
    v = torch.randn(B, 1, S, Dv, device=device, dtype=dtype, requires_grad=True)
    qi = torch.randn(B, S, Hi, Di, device=device, dtype=dtype, requires_grad=True)
    ki = torch.randn(B, S, 1, Di, device=device, dtype=dtype, requires_grad=True)
    w = torch.rand(B, S, Hi, device=device, requires_grad=True)
    return q, k, v, qi, ki, w


def test_fused_dsa_matches_eager_oracle_cpu():
    from titan_b200.models.deepseek_v32.model import DSASparseAttention
    from titan_b200.ops.dsa import dsa_attention

    q, k, v, qi, ki, w = _inputs()
    loss_ref, out_ref = DSASparseAttention()(q, k, v, scale=0.2, q_indexer=qi, k_indexer=ki, weights=w, index_topk=8)
    ins2 = [t.detach().clone().requires_grad_() for t in (q, k, v, qi, ki, w)]
    loss, out = dsa_attention(ins2[0], ins2[1], ins2[2], scale=0.2, q_indexer=ins2[3], k_indexer=ins2[4],
                              weights=ins2[5], index_topk=8)
    torch.testing.assert_close(out, out_ref, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(loss, loss_ref, rtol=1e-4, atol=1e-6)
    (out_ref.sum() + loss_ref).backward()
    (out.sum() + loss).backward()
    for a, b, name in zip(ins2, (q, k, v, qi, ki, w), "q k v qi ki w".split()):
        torch.testing.assert_close(a.grad, b.grad, rtol=1e-3, atol=1e-5, msg=f"grad of {name}")


def test_indexer_topk_ref_padding():
    from titan_b200.ops.dsa import lightning_indexer_topk_ref

    _, _, _, qi, ki, w = _inputs(S=6)
    idx, vals = lightning_indexer_topk_ref(qi, w, ki, topk=4)
    assert idx.shape == (1, 6, 4)
    assert (idx[0, 0] == torch.tensor([0, -1, -1, -1])).all()  # the first query sees one key
    assert torch.isinf(vals[0, 0, 1:]).all() and (idx[0, 5] >= 0).all()


def test_dsa_converter_swaps_core():
    from titan_b200.converters.dsa import FusedDSAttention
    from titan_b200.models.deepseek_v32 import deepseekv32_configs
    from titan_b200.protocols import converter as conv

    m = deepseekv32_configs["smoketest"]().build()
    conv.ModelConvertersContainer([conv.get_model_converter_config("npu_dsa")]).convert(m)
    assert isinstance(m.layers["0"].attention.inner_attention, FusedDSAttention)
    m.init_states()
    out = m(torch.randint(0, 2048, (1, 64)))
    assert torch.isfinite(out).all()


@pytest.mark.gpu
@pytest.mark.parametrize("S,H,T,k,off", [(300, 64, 300, 64, 0), (128, 4, 640, 100, 512), (1000, 64, 1000, 2048, 0)])
def test_indexer_kernels_match_reference(cuda_device, S, H, T, k, off):
    from titan_b200.ops import _lib
    from titan_b200.ops.dsa import lightning_indexer_topk, lightning_indexer_topk_ref

    torch.manual_seed(0)
    qi = torch.randn(1, S, H, 128, device="cuda", dtype=torch.bfloat16)
    ki = torch.randn(1, T, 1, 128, device="cuda", dtype=torch.bfloat16)
    w = torch.rand(1, S, H, device="cuda")
    idx, vals = lightning_indexer_topk(qi, w, ki, k, off)
    _lib.shared_status().raise_if_set("indexer")
    idx_r, vals_r = lightning_indexer_topk_ref(qi, w, ki, k, off)
    # same selected SET per row (order is free); compare through sorted values and index sets on clear margins
    sv, _ = vals.sort(-1, descending=True)
    sr, _ = vals_r.sort(-1, descending=True)
    finite = torch.isfinite(sr)
    torch.testing.assert_close(sv[finite], sr[finite], rtol=2e-2, atol=2e-1)
    assert ((idx >= 0).sum(-1) == (idx_r >= 0).sum(-1)).all()
    pos = torch.arange(S, device="cuda").view(1, S, 1) + off
    assert ((idx <= pos) | (idx < 0)).all()  # causality
    overlap = []
    for s in range(0, S, max(S // 16, 1)):
        a, b = set(idx[0, s].tolist()) - {-1}, set(idx_r[0, s].tolist()) - {-1}
        overlap.append(len(a & b) / max(len(b), 1))
    assert min(overlap) > 0.9  # bf16 rounding may swap a few keys at the threshold


def test_sparse_mla_dense_mask_and_gather_paths_agree():
    """Selected keys through one masked GEMM (short key streams) or through a row gather with a scatter-add backward
    (long ones): same outputs, same gradients; the same for the differentiable index scores."""
    from titan_b200.ops import dsa

    torch.manual_seed(5)
    B, H, S, Dq, Dv, k = 1, 2, 24, 8, 6, 5
    mk = lambda *s: torch.randn(*s, dtype=torch.float64)
    q, kk, v = mk(B, H, S, Dq), mk(B, 1, S, Dq), mk(B, 1, S, Dv)
    qi, ki, w = mk(B, S, 3, 4), mk(B, S, 1, 4), torch.rand(B, S, 3, dtype=torch.float64)
    idx = torch.full((B, S, k), -1, dtype=torch.long)
    for s in range(S):
        pick = torch.randperm(s + 1)[:k]
        idx[0, s, : pick.numel()] = pick
    results = []
    saved = dsa.DENSE_RATIO
    for ratio in (4, 0):
        dsa.DENSE_RATIO = ratio
        try:
            leaves = [t.clone().requires_grad_(True) for t in (q, kk, v, qi, ki, w)]
            out, teacher, lse = dsa.sparse_mla_attention(leaves[0], leaves[1], leaves[2], idx, Dq ** -0.5, chunk=8)
            sc = dsa.indexer_scores_selected(leaves[3], leaves[5], leaves[4], idx, chunk=8)
            (out.square().sum() + sc.masked_fill(idx < 0, 0.0).sum()).backward()
            results.append((out.detach(), teacher, lse.detach(), sc.detach(), [t.grad for t in leaves]))
        finally:
            dsa.DENSE_RATIO = saved
    a, b = results
    for x, y in zip(a[:4], b[:4]):
        torch.testing.assert_close(x, y)
    for x, y in zip(a[4], b[4]):  # the gather path accumulates its scatter-add in fp32
        torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,T", [(torch.bfloat16, 64), (torch.bfloat16, 8192), (torch.bfloat16, 16384),
                                     (torch.bfloat16, 40960), (torch.float32, 1024), (torch.float32, 8192),
                                     (torch.float32, 16384)])
def test_masked_softmax_kernel_matches_reference(cuda_device, dtype, T):
    from titan_b200.ops.masked_softmax import masked_softmax, masked_softmax_ref

    torch.manual_seed(0)
    H, Sc = 3, 40
    s = (torch.randn(H, Sc, T, device="cuda") * 4).to(dtype)
    allowed = torch.rand(Sc, T, device="cuda") < 0.3
    allowed[5] = False  # a query without any visible key
    a, b = s.clone().requires_grad_(True), s.clone().requires_grad_(True)
    sink = torch.randn(H, device="cuda") if T % 3 == 1 else None  # some cases with an attention sink
    sa = sink.clone().requires_grad_(True) if sink is not None else None
    sb = sink.clone().requires_grad_(True) if sink is not None else None
    p, ref = masked_softmax(a, allowed, 0.7, sa), masked_softmax_ref(b, allowed, 0.7, sb)
    tol = dict(rtol=2e-2, atol=2e-3) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(p.float(), ref.float(), **tol)
    assert p[:, 5].abs().sum() == 0
    g = torch.randn_like(p)
    p.backward(g)
    ref.backward(g)
    gtol = dict(rtol=5e-2, atol=5e-3) if dtype == torch.bfloat16 else dict(rtol=1e-3, atol=1e-5)
    torch.testing.assert_close(a.grad.float(), b.grad.float(), **gtol)
    if sink is not None:
        torch.testing.assert_close(sa.grad, sb.grad, rtol=5e-2, atol=5e-2)


@pytest.mark.gpu
def test_indexer_scores_from_selection_match_recomputed_scores(cuda_device):
    """Forward values come from the scoring kernel, the backward from one fused kernel + GEMMs: both against the
    PyTorch scores recomputed at the selected keys."""
    from titan_b200.ops import dsa

    torch.manual_seed(1)
    B, S, H, D, T, k = 1, 300, 8, 32, 512, 64
    q = (torch.randn(B, S, H, D, device="cuda") * 0.5).to(torch.bfloat16)
    kk = (torch.randn(B, T, 1, D, device="cuda") * 0.5).to(torch.bfloat16)
    w = torch.rand(B, S, H, device="cuda")
    idx, vals = dsa.lightning_indexer_topk(q, w, kk, k, T - S)
    a = [t.clone().requires_grad_(True) for t in (q, w, kk)]
    b = [t.clone().requires_grad_(True) for t in (q, w, kk)]
    got = dsa.indexer_scores_from_selection(a[0], a[1], a[2], idx, vals, chunk=128)
    ref = dsa.indexer_scores_selected(b[0], b[1], b[2], idx)
    m = idx >= 0
    torch.testing.assert_close(got[m], ref[m], rtol=2e-2, atol=2e-2)
    g = torch.randn_like(ref).masked_fill(~m, 0.0)
    got.masked_fill(~m, 0.0).mul(g).sum().backward()
    ref.masked_fill(~m, 0.0).mul(g).sum().backward()
    for x, y, name in zip(a, b, ("dq", "dw", "dk")):
        torch.testing.assert_close(x.grad.float(), y.grad.float(), rtol=5e-2, atol=5e-2, msg=lambda s, n=name: f"{n}: {s}")


@pytest.mark.gpu
@pytest.mark.parametrize("S,H,T,k", [(70, 64, 1024, 256), (33, 16, 400, 100), (16, 32, 2048, 384)])
def test_selected_key_indexer_backward_kernel(cuda_device, S, H, T, k):
    """The tensor-core backward through the selected keys only (head dim 128; 16 / 32 / 64 index heads; top-k that is
    and is not a multiple of 128; empty slots) against fp32 autograd of the scores recomputed at the selected keys."""
    from titan_b200.ops import _lib, dsa

    torch.manual_seed(5)
    B, D = 2, 128
    q = (torch.randn(B, S, H, D, device="cuda") * 0.3).to(torch.bfloat16)
    kk = (torch.randn(B, T, 1, D, device="cuda") * 0.3).to(torch.bfloat16)
    w = torch.rand(B, S, H, device="cuda")
    idx = torch.stack([torch.stack([torch.randperm(T, device="cuda")[:k] for _ in range(S)]) for _ in range(B)])
    idx = torch.where(torch.rand(B, S, k, device="cuda") < 0.15, torch.full_like(idx, -1), idx).to(torch.int32)
    assert dsa._selected_backward_takes(q, kk)
    # fp32 oracle: scores at the selected keys
    qr, wr, kr = q.float().requires_grad_(), w.clone().requires_grad_(), kk.float().requires_grad_()
    ksel = torch.stack([kr[b, :, 0][idx[b].clamp_min(0).long()] for b in range(B)])          # [B,S,k,D]
    x = torch.einsum("bshd,bskd->bshk", qr, ksel)
    ref = (torch.relu(x) * wr.unsqueeze(-1)).sum(2)
    vals = ref.detach().masked_fill(idx < 0, float("-inf"))
    a = [t.clone().requires_grad_(True) for t in (q, w, kk)]
    got = dsa.indexer_scores_from_selection(a[0], a[1], a[2], idx, vals)
    m = idx >= 0
    g = torch.randn_like(ref).masked_fill(~m, 0.0)
    got.masked_fill(~m, 0.0).mul(g).sum().backward()
    _lib.shared_status().raise_if_set("indexer_sel_bwd")
    ref.masked_fill(~m, 0.0).mul(g).sum().backward()
    for xg, y, name in zip(a, (qr, wr, kr), ("dq", "dw", "dk")):
        torch.testing.assert_close(xg.grad.float(), y.grad.float(), rtol=5e-2, atol=5e-2,
                                   msg=lambda s_, n=name: f"{n}: {s_}")


@pytest.mark.gpu
@pytest.mark.parametrize("S,H,T,k,off,ratio", [(257, 64, 900, 128, 643, 1), (130, 16, 512, 64, 0, 1),
                                               (96, 256, 300, 32, 204, 1), (512, 32, 128, 40, 0, 4)])
def test_resident_query_scoring_kernel_matches_the_tiled_gemm_form(cuda_device, S, H, T, k, off, ratio):
    """Head dim 128 takes the kernel that keeps a block of 256 (query, head) rows in shared memory and streams the
    key tiles past it; the generic tiled GEMM's indexer mode is the oracle (same bf16 inputs, fp32 sums): equal
    selected values, equal selections up to ties, for several head counts, offsets and a compression ratio."""
    from titan_b200.ops import _lib, dsa

    torch.manual_seed(4)
    qi = torch.randn(1, S, H, 128, device="cuda", dtype=torch.bfloat16)
    ki = torch.randn(1, T, 1, 128, device="cuda", dtype=torch.bfloat16)
    w = torch.rand(1, S, H, device="cuda")
    idx, vals = dsa.lightning_indexer_topk(qi, w, ki, k, off, ratio)
    _lib.shared_status().raise_if_set("indexer_scores_resident")
    saved = dsa.RESIDENT_SCORING
    dsa.RESIDENT_SCORING = False
    try:
        idx_r, vals_r = dsa.lightning_indexer_topk(qi, w, ki, k, off, ratio)
    finally:
        dsa.RESIDENT_SCORING = saved
    assert ((idx >= 0) == (idx_r >= 0)).all()
    sv, sr = vals.sort(-1, descending=True)[0], vals_r.sort(-1, descending=True)[0]
    finite = torch.isfinite(sr)
    torch.testing.assert_close(sv[finite], sr[finite], rtol=1e-4, atol=1e-3)
    same = (idx.sort(-1)[0] == idx_r.sort(-1)[0]).float().mean()
    assert same > 0.98
