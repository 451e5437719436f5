"""DeepSeek sparse attention (DSA) operators.

* `lightning_indexer_topk` – index scores ``Σ_h w[s,h]·relu(q_idx[s,h]·k_idx[t])`` for every visible key and
  the top-k keys per query.  On CUDA the S×T scoring runs on the tcgen05 GEMM with a fused
  relu·weight·head-sum epilogue (`tb_indexer_scores`; tiles in the causal future are skipped) and selection
  is an exact radix select (`tb_topk_select`); nothing of size ``[S, T]`` per head is ever materialised.
  Selection carries no gradient.
* `sparse_mla_attention`   – attention of every query over its selected keys of the shared one-head KV latent
  (MLA absorb layout), in query chunks: gather ``[chunk, k, D]`` rows → scores → softmax (+ log-sum-exp) →
  values.  Also returns the head-summed probability mass on the selected keys (the indexer's teacher).
* `indexer_scores_selected` – differentiable re-evaluation of the index scores at the selected keys only
  (``O(S·k)``): this is where the indexer's parameters get their gradient.
* `dsa_attention`           – the three together + the KL indexer loss; the drop-in for the eager oracle.

Parity: `npu_lightning_indexer`, `npu_sparse_flash_attention`, `npu_sparse_lightning_indexer_grad_kl_loss`
(torchtitan_npu/converters/kernels/dsa.py:22-309) with the eager model code as oracle
(models/deepseek_v32/model.py:224-236, 363-420).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from titan_b200.models.common.dsa_indexer_loss import dsa_indexer_loss
from titan_b200.ops import _lib

__all__ = ["lightning_indexer_topk", "lightning_indexer_topk_ref", "sparse_mla_attention",
           "indexer_scores_selected", "dsa_attention"]


def lightning_indexer_topk_ref(q_idx, weights, k_idx, topk: int, pos_offset: int = 0, ratio: int = 1):
    """Oracle: dense scores, causal mask, `torch.topk`; invalid slots → index -1 / value -inf."""
    B, S, H, D = q_idx.shape
    T = k_idx.shape[1]
    p = torch.matmul(q_idx.float().transpose(1, 2), k_idx.float().permute(0, 2, 3, 1))
    score = (F.relu(p) * weights.float().permute(0, 2, 1).unsqueeze(-1)).sum(1)  # [B, S, T]
    visible = (torch.arange(S, device=score.device).unsqueeze(-1) + pos_offset + 1) // ratio
    future = torch.arange(T, device=score.device).unsqueeze(0) >= visible
    score = score.masked_fill(future, float("-inf"))
    kk = min(topk, T)
    vals, idx = score.topk(kk, dim=-1)
    valid = torch.isfinite(vals)
    idx = torch.where(valid, idx, torch.full_like(idx, -1))
    if kk < topk:
        idx = F.pad(idx, (0, topk - kk), value=-1)
        vals = F.pad(vals, (0, topk - kk), value=float("-inf"))
    return idx.to(torch.int32), vals


def _scoring_kernels_take(q_idx) -> bool:
    heads = q_idx.shape[2]
    return ((q_idx.is_cuda or q_idx.is_meta) and q_idx.dtype in (torch.bfloat16, torch.float16) and heads <= 256
            and heads & (heads - 1) == 0 and q_idx.shape[3] % 8 == 0)


@torch.no_grad()
def lightning_indexer_topk(q_idx, weights, k_idx, topk: int, pos_offset: int = 0, ratio: int = 1):
    """q_idx [B,S,H,D], weights [B,S,H], k_idx [B,T,1,D] → (idx [B,S,topk] int32 with -1 padding, vals fp32).

    ``ratio`` > 1: the keys are compressed blocks of ``ratio`` tokens; query ``s`` sees the first
    ``(pos_offset + s + 1) // ratio`` of them."""
    if not _scoring_kernels_take(q_idx):
        return lightning_indexer_topk_ref(q_idx, weights, k_idx, topk, pos_offset, ratio)
    from titan_b200.ops.registry import ops

    # a dispatcher op: selective activation checkpointing keeps the selection instead of scoring every key again
    return ops.indexer_topk(q_idx.detach(), weights.detach(), k_idx.detach(), topk, pos_offset, ratio)


RESIDENT_SCORING = True  # False: the generic tiled GEMM's indexer mode for every shape (the oracle of the other's test)


def _indexer_topk_launch(q_idx, weights, k_idx, topk: int, pos_offset: int = 0, ratio: int = 1):
    B, S, H, D = q_idx.shape
    T = k_idx.shape[1]
    L = _lib.lib()
    import ctypes

    P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    _lib.declare("tb_indexer_scores", [P, P, P, P, I, I, I, I, LL, I, I, I, P, P])
    _lib.declare("tb_topk_select", [P, LL, I, I, I, I, I, P, P, P])
    _lib.declare("tb_indexer_scores_resident", [P, P, P, P, I, I, I, I, LL, I, I, P, P])
    ld = (T + 3) // 4 * 4
    scores = torch.empty(S, ld, dtype=torch.float32, device=q_idx.device)
    idx = torch.empty(B, S, topk, dtype=torch.int32, device=q_idx.device)
    vals = torch.empty(B, S, topk, dtype=torch.float32, device=q_idx.device)
    for b in range(B):
        q2 = q_idx[b].reshape(S * H, D).contiguous()
        k2 = k_idx[b].reshape(T, D).contiguous().to(q2.dtype)
        w2 = weights[b].reshape(S * H).float().contiguous()
        if RESIDENT_SCORING and D == 128 and q2.dtype == torch.bfloat16 and 16 <= H <= 256 and (H & (H - 1)) == 0:
            # head dim 128: the query block stays in shared memory and key tiles stream past it
            rc = L.tb_indexer_scores_resident(q2.data_ptr(), k2.data_ptr(), w2.data_ptr(), scores.data_ptr(), S, H, T,
                                              D, ld, pos_offset, ratio, _lib.shared_status().ptr, _lib.stream_ptr())
        else:
            rc = L.tb_indexer_scores(q2.data_ptr(), k2.data_ptr(), w2.data_ptr(), scores.data_ptr(), S, H, T, D, ld,
                                     pos_offset, ratio, _lib.dtype_code(q2.dtype), _lib.shared_status().ptr,
                                     _lib.stream_ptr())
        _lib.check(rc, "indexer_scores")
        rc = L.tb_topk_select(scores.data_ptr(), ld, S, T, topk, pos_offset, ratio, idx[b].data_ptr(),
                              vals[b].data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "topk_select")
    return idx, vals


DENSE_RATIO = 64  # a key stream at most this many times longer than top-k is scored densely with a selection mask


class _GatherRows(torch.autograd.Function):
    """``src[idx]`` for ``src [T, D]`` and integer ``idx [...]``; the backward is ONE scatter-add with fp32 atomics
    (the stock advanced-indexing backward sorts the indices first: 68 % of a DeepSeek-V4 step when it was used here)."""

    @staticmethod
    def forward(ctx, src, idx):
        ctx.save_for_backward(idx)
        ctx.rows, ctx.dtype = src.shape[0], src.dtype
        return src[idx]

    @staticmethod
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        d = g.shape[-1]
        acc = torch.zeros(ctx.rows, d, dtype=torch.float32, device=g.device)
        acc.index_add_(0, idx.reshape(-1), g.reshape(-1, d).float())
        return acc.to(ctx.dtype), None


def gather_rows(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    return _GatherRows.apply(src, idx)


def _dense_index_scores(q, w, k, safe):
    """q [Sc,H,D], w [Sc,H], k [T,D], safe [Sc,kk] → scores of the selected keys [Sc,kk] through one GEMM."""
    s = torch.einsum("shd,td->sht", q, k).float()
    s = (F.relu(s) * w.float().unsqueeze(-1)).sum(1)  # [Sc,T]
    return torch.gather(s, 1, safe)


def indexer_scores_selected(q_idx, weights, k_idx, idx, chunk: int = 512):
    """Differentiable index scores at the selected keys: [B,S,k]; padded slots (-1) → -inf.  A short key stream is
    scored densely in query chunks (one GEMM, then a gather along the key axis); a long one gathers the selected key
    rows (scatter-add backward)."""
    B, S, H, D = q_idx.shape
    T, kk = k_idx.shape[1], idx.shape[-1]
    safe = idx.clamp_min(0).long()
    if T <= DENSE_RATIO * kk:
        need_grad = torch.is_grad_enabled() and (q_idx.requires_grad or k_idx.requires_grad or weights.requires_grad)
        rows = []
        for b in range(B):
            parts = []
            for s0 in range(0, S, chunk):
                args = (q_idx[b, s0:s0 + chunk], weights[b, s0:s0 + chunk], k_idx[b, :, 0], safe[b, s0:s0 + chunk])
                parts.append(checkpoint(_dense_index_scores, *args, use_reentrant=False) if need_grad
                             else _dense_index_scores(*args))
            rows.append(torch.cat(parts, dim=0))
        s = torch.stack(rows)
    else:
        ksel = torch.stack([gather_rows(k_idx[b, :, 0], safe[b]) for b in range(B)])  # [B,S,k,D]
        s = torch.einsum("bshd,bskd->bshk", q_idx.float(), ksel.float())
        s = (F.relu(s) * weights.float().unsqueeze(-1)).sum(2)
    return s.masked_fill(idx < 0, float("-inf"))


class _IndexScoresAtSelected(torch.autograd.Function):
    """Index scores at the selected keys whose forward costs nothing (the scoring kernel already produced the values
    while selecting).  The gradient only flows through the selected keys, so the backward gathers those key rows and
    runs on the tensor cores in O(S * top-k) (`csrc/attention/indexer_sel_bwd.cu`); other shapes take a dense pass
    over all keys in query chunks."""

    @staticmethod
    def forward(ctx, q_idx, weights, k_idx, idx, vals, chunk):
        ctx.save_for_backward(q_idx, weights, k_idx, idx)
        ctx.chunk = chunk
        return vals.float().masked_fill(idx < 0, float("-inf"))

    @staticmethod
    def backward(ctx, g):
        q_idx, weights, k_idx, idx = ctx.saved_tensors
        g = g.float().masked_fill(idx < 0, 0.0)
        if SELECTED_BACKWARD and _selected_backward_takes(q_idx, k_idx):
            dq, dw, dk = _indexer_selected_backward(q_idx, weights, k_idx, idx, g)
        else:
            dq, dw, dk = _indexer_dense_backward(q_idx, weights, k_idx, idx, g, ctx.chunk)
        return dq, dw.to(weights.dtype), dk.to(k_idx.dtype).unsqueeze(2), None, None, None


SELECTED_BACKWARD = True  # False: the dense chunked backward below (the oracle of the sparse kernel's test)


def _selected_backward_takes(q_idx, k_idx) -> bool:
    return ((q_idx.is_cuda or q_idx.is_meta) and q_idx.dtype == torch.bfloat16 and q_idx.shape[-1] == 128
            and q_idx.shape[2] in (16, 32, 64))


def _indexer_selected_backward(q_idx, weights, k_idx, idx, g):
    """Gradients through the selected keys only (`csrc/attention/indexer_sel_bwd.cu`): O(S * top-k) work.
    → (dq like q_idx, dw [B,S,H] fp32, dk [B,T,D] fp32)."""
    import ctypes

    B, S, H, D = q_idx.shape
    T, kk = k_idx.shape[1], idx.shape[-1]
    P, I = ctypes.c_void_p, ctypes.c_int
    meta = q_idx.is_meta   # shapes only (memory simulation): same buffers, no launches
    if not meta:
        _lib.declare("tb_indexer_sel_bwd", [P, P, P, P, P, P, P, P, I, I, I, I, I, P, P])
    pad = (-kk) % 128
    if pad:
        idx, g = F.pad(idx, (0, pad), value=-1), F.pad(g, (0, pad))
    idx = idx.to(torch.int32).contiguous()
    g = g.contiguous()
    dq = torch.empty_like(q_idx, memory_format=torch.contiguous_format)
    dw = torch.empty(B, S, H, dtype=torch.float32, device=q_idx.device)
    dk = torch.zeros(B, T, D, dtype=torch.float32, device=q_idx.device)
    for b in range(B):
        qb = q_idx[b].contiguous()
        kb = k_idx[b, :, 0].contiguous().to(qb.dtype)
        wb = weights[b].float().contiguous()
        if meta:
            _lib.note_skipped_launch("tb_indexer_sel_bwd", (None,) * 8 + (S, H, T, kk + pad, D))
            continue
        rc = _lib.lib().tb_indexer_sel_bwd(qb.data_ptr(), kb.data_ptr(), idx[b].data_ptr(), g[b].data_ptr(),
                                           wb.data_ptr(), dq[b].data_ptr(), dw[b].data_ptr(), dk[b].data_ptr(),
                                           S, H, T, kk + pad, D, _lib.shared_status().ptr, _lib.stream_ptr())
        _lib.check(rc, "indexer_sel_bwd")
    return dq, dw, dk


def _indexer_dense_backward(q_idx, weights, k_idx, idx, g, chunk):
    """The same gradients through a dense pass over all keys, ``chunk`` queries at a time: recompute ``x = q·kᵀ`` in
    the storage dtype, one kernel for ``dx`` and ``dw`` (`csrc/attention/indexer_bwd.cu`), two GEMMs for ``dq`` /
    ``dk``.  Never builds fp32 [queries, heads, keys] tensors."""
    import ctypes

    B, S, H, D = q_idx.shape
    T = k_idx.shape[1]
    P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    meta = q_idx.is_meta   # shapes only (memory simulation): same buffers, no launches
    if not meta:
        _lib.declare("tb_indexer_relu_bwd", [P, P, P, P, P, LL, I, I, I, P])
    safe = idx.clamp_min(0).long()
    dq = torch.empty_like(q_idx)
    dw = torch.empty(B, S, H, dtype=torch.float32, device=q_idx.device)
    dk = torch.zeros(B, T, D, dtype=torch.float32, device=q_idx.device)
    for b in range(B):
        kb = k_idx[b, :, 0].contiguous()
        for s0 in range(0, S, chunk):
            s1 = min(s0 + chunk, S)
            sc = s1 - s0
            qc = q_idx[b, s0:s1].reshape(sc * H, D)
            dense_g = torch.zeros(sc, T, dtype=torch.float32, device=g.device).scatter_add_(1, safe[b, s0:s1],
                                                                                        g[b, s0:s1])
            x = torch.matmul(qc, kb.t())  # [sc*H, T], storage dtype
            dx = torch.empty_like(x)
            dwc = torch.empty(sc * H, dtype=torch.float32, device=x.device)
            wc = weights[b, s0:s1].float().contiguous()
            if not meta:
                rc = _lib.lib().tb_indexer_relu_bwd(x.data_ptr(), dense_g.data_ptr(), wc.data_ptr(), dx.data_ptr(),
                                                    dwc.data_ptr(), sc * H, H, T, _lib.dtype_code(x.dtype),
                                                    _lib.stream_ptr())
                _lib.check(rc, "indexer_relu_bwd")
            dq[b, s0:s1] = torch.matmul(dx, kb).view(sc, H, D)
            dk[b] += torch.matmul(dx.t(), qc).float()
            dw[b, s0:s1] = dwc.view(sc, H)
    return dq, dw, dk


def indexer_scores_from_selection(q_idx, weights, k_idx, idx, vals, chunk: int = 256):
    """Differentiable scores at the selected keys, given the values the selection kernels already computed."""
    return _IndexScoresAtSelected.apply(q_idx, weights, k_idx, idx, vals, chunk)


def _sparse_chunk(q, kv, v, idx, scale, want_lse=True):
    """q [H,Sc,Dq], kv [T,Dq], v [T,Dv], idx [Sc,k] → (out [H,Sc,Dv], teacher [Sc,k], lse [H,Sc]); without
    ``want_lse`` the dense path skips the extra pass over the logits and returns zeros there."""
    safe = idx.clamp_min(0).long()
    T = kv.shape[0]
    if T <= DENSE_RATIO * idx.shape[1]:
        # short key stream: every key through one GEMM, the selection as a mask (no gather, no scatter-add)
        # the GEMMs stay in the storage dtype (bf16 tensor cores; an fp32 copy of the operands would run them as TF32
        # at half the rate and move twice the bytes); softmax statistics are fp32.  The [H,Sc,T] logits are touched by
        # as few passes as possible: scale folded into q, mask and softmax in one kernel.
        slot = torch.where(idx < 0, T, idx).long()
        allowed = torch.zeros(idx.shape[0], T + 1, dtype=torch.bool, device=q.device).scatter_(1, slot, True)[:, :T]
        from titan_b200.ops.masked_softmax import masked_softmax

        s = torch.matmul(q * scale, kv.t())  # [H,Sc,T] in the storage dtype
        p = masked_softmax(s, allowed)       # one kernel: mask + fp32 softmax, rows without a visible key -> zeros
        with torch.no_grad():
            if want_lse:
                lse = torch.logsumexp(s.float().masked_fill(~allowed.unsqueeze(0), float("-inf")), dim=-1)
            else:
                lse = s.new_zeros(s.shape[:2], dtype=torch.float32)
        out = torch.matmul(p.to(v.dtype), v).to(q.dtype)
        teacher = torch.gather(p.detach().sum(0, dtype=torch.float32), 1, safe).masked_fill(idx < 0, 0.0)
        return out, teacher, lse
    ksel, vsel = gather_rows(kv, safe), gather_rows(v, safe)  # [Sc,k,D]
    s = torch.einsum("hsd,skd->hsk", q.float(), ksel.float()) * scale
    s = s.masked_fill((idx < 0).unsqueeze(0), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p)  # a row without any visible key
    out = torch.einsum("hsk,skd->hsd", p, vsel.float()).to(q.dtype)
    return out, p.detach().sum(0), lse


KERNEL_RATIO = 4  # key streams at least this many times top-k go to the gathered-tile tensor-core kernel


def _values_are_key_prefix(k: torch.Tensor, v: torch.Tensor) -> bool:
    """MLA absorb layout: the values are the latent part of the keys (``v == k[..., :Dv]``).  Checked on a few rows
    (one small device-to-host read; callers cache the answer per module)."""
    if v.shape[-1] > k.shape[-1] or v.shape[:-1] != k.shape[:-1]:
        return False
    if k.is_meta:
        return True   # shapes only (memory simulation): the absorb layout is the one that passes the shape test
    dv, t = v.shape[-1], k.shape[2]
    rows = sorted({0, t // 2, t - 1})
    with torch.no_grad():   # a probe, not part of the graph (under activation checkpointing it runs only once)
        kd, vd = k.detach(), v.detach()
        return bool(torch.equal(kd[0, 0, rows, :dv], vd[0, 0, rows]))


def _kernel_sparse_attention(q, k, idx, scale, dv):
    """The tcgen05 sparse kernel per batch row → (out [B,H,S,Dv], teacher [B,S,topk], lse [B,H,S])."""
    from titan_b200.ops.sparse_mla import sparse_mla

    B, topk = q.shape[0], idx.shape[-1]
    pad = (-topk) % 128
    outs, teach, lses = [], [], []
    for b in range(B):
        ib = F.pad(idx[b], (0, pad), value=-1) if pad else idx[b]
        o, t, l = sparse_mla(q[b].transpose(0, 1).contiguous(), k[b, 0], ib, scale, dv)
        outs.append(o.transpose(0, 1)); teach.append(t[:, :topk]); lses.append(l.t())
    return torch.stack(outs), torch.stack(teach), torch.stack(lses)


def sparse_mla_attention(q, k, v, idx, scale: float, chunk: int = 256, want_lse: bool = True,
                         values_are_key_prefix: bool | None = None):
    """q [B,H,S,Dq], k [B,1,T,Dq], v [B,1,T,Dv], idx [B,S,topk] → (out [B,H,S,Dv], teacher [B,S,topk], lse [B,H,S]).

    Long key streams (at least `KERNEL_RATIO` x top-k keys) in the MLA absorb layout run on the gathered-tile
    tensor-core kernel (`titan_b200.ops.sparse_mla`): work and memory O(S * top-k).  ``values_are_key_prefix`` says
    that ``v`` is the latent part of ``k`` (None = check a few rows)."""
    B, H, S, _ = q.shape
    T, dv = k.shape[2], v.shape[-1]
    if T >= KERNEL_RATIO * idx.shape[-1] and (q.is_cuda or q.is_meta):
        from titan_b200.ops.sparse_mla import sparse_mla_supported

        if sparse_mla_supported(q[0].transpose(0, 1), k[0, 0], F.pad(idx[0], (0, (-idx.shape[-1]) % 128)), dv):
            if values_are_key_prefix is None:
                values_are_key_prefix = _values_are_key_prefix(k, v)
            if values_are_key_prefix:
                return _kernel_sparse_attention(q, k, idx, scale, dv)
    outs, teach, lses = [], [], []
    for b in range(B):
        ob, tb, lb = [], [], []
        for s0 in range(0, S, chunk):
            s1 = min(s0 + chunk, S)
            args = (q[b, :, s0:s1], k[b, 0], v[b, 0], idx[b, s0:s1], scale, want_lse)
            if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad):
                o, t, l = checkpoint(_sparse_chunk, *args, use_reentrant=False)  # gathered rows are not kept
            else:
                o, t, l = _sparse_chunk(*args)
            ob.append(o); tb.append(t); lb.append(l)
        outs.append(torch.cat(ob, dim=1)); teach.append(torch.cat(tb, dim=0)); lses.append(torch.cat(lb, dim=1))
    return torch.stack(outs), torch.stack(teach), torch.stack(lses)


def dsa_attention(q, k, v, *, scale, q_indexer, k_indexer, weights, index_topk: int, loss_scale: float = 1.0,
                  values_are_key_prefix: bool | None = None):
    """Fused-path equivalent of the eager sparse-attention oracle → (indexer loss, out [B,H,S,Dv])."""
    S, T = q.shape[2], k.shape[2]
    pos_offset = T - S  # with context parallelism the local queries are the tail of the gathered key range
    topk = min(index_topk, T)
    idx, vals = lightning_indexer_topk(q_indexer, weights, k_indexer, topk, pos_offset)
    out, teacher, _ = sparse_mla_attention(q, k, v, idx, scale, want_lse=False,
                                           values_are_key_prefix=values_are_key_prefix)
    if _scoring_kernels_take(q_indexer) and T % 8 == 0:
        student = indexer_scores_from_selection(q_indexer, weights, k_indexer, idx, vals)
    else:
        student = indexer_scores_selected(q_indexer, weights, k_indexer, idx)
    student = torch.where(idx < 0, torch.full_like(student, -1e30), student)  # finite: masked slots get zero mass
    loss = dsa_indexer_loss(teacher.masked_fill(idx < 0, 0.0), student, loss_scale)
    return loss, out
