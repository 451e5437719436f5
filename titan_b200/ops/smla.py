"""Sparse multi-query latent attention for DeepSeek-V4: sliding window ∪ compressed keys ∪ sink.

Every query attends to
* its causal window of ``window`` raw keys of the one shared KV latent (values = keys),
* compressed keys: either the ``k`` picked by the lightning indexer (``compress_idx``, ratio 4) or every compressed
  key whose block is complete (other ratios),
* a learned per-head sink logit that takes probability mass and contributes no value.

`smla_attention` never builds anything of size ``S × T``: queries are processed in chunks; a chunk touches the
``chunk + window`` raw keys it can see (dense band) and gathers its selected compressed keys.  Chunks are
recomputed in backward, so what stays alive is O(S·H·hd).  It also returns the head-mean probability on the selected
compressed keys – the teacher of the indexer's KL loss – so the loss needs no second attention pass.

`li_select` is the matching selection step: tcgen05 index scoring + radix top-k over the compressed keys, then a
differentiable re-evaluation of the scores at the selected keys only (that is where the indexer gets its gradient).

Parity: `SparseAttention`, `LiCompute`, `LiLoss._current_selected_attn_dist`
(torchtitan_npu/models/deepseek_v4/model.py:421-457, 553-657) and the fused `npu_smla` path
(converters/kernels/npu_smla.py).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

__all__ = ["smla_attention", "li_select"]


from titan_b200.ops import _lib
from titan_b200.ops.dsa import gather_rows

DENSE_RATIO = 64  # a compressed stream at most this many times longer than k is attended densely with a mask
KERNEL_RATIO = 4  # compressed streams longer than this many times the selection go to the gathered-tile kernel


def _kernel_takes(q, kv_compress, compress_idx, window: int, ratio: int) -> bool:
    """The gathered-tile tensor-core kernel (`titan_b200.ops.sparse_mla`) serves window + selected compressed keys +
    sink when the head dim is a multiple of 128 (keys are values here: dq = dv = hd) and the compressed stream is long
    compared with what a query actually attends to."""
    hd, H = q.shape[-1], q.shape[2]
    if not (_lib.on_device(q) and q.dtype == torch.bfloat16 and H % 16 == 0 and hd % 128 == 0 and hd <= 512):
        return False
    if kv_compress is None or ratio <= 1:
        return False
    k = compress_idx.shape[-1] if compress_idx is not None else kv_compress.shape[1]
    return compress_idx is not None and kv_compress.shape[1] > KERNEL_RATIO * max(k, 128)


def _smla_kernel_row(q, kv, sink, kvc, cidx, koff: int, window: int, scale: float, n_heads_total: int,
                     want_dist: bool):
    """One batch row through the sparse kernel.  q [S,H,hd]; kv [Tk,hd] raw keys (local query s sits at key s + koff);
    kvc [Tc,hd]; cidx [S,k] ids into kvc (-1 = empty).  The keys of a query are listed explicitly: its window of raw
    keys followed by its selected compressed keys, as rows of ONE buffer [raw keys ; compressed keys]."""
    from titan_b200.ops.sparse_mla import sparse_mla

    S, H, hd = q.shape
    Tk, k = kv.shape[0], cidx.shape[1]
    pos = torch.arange(S, device=q.device).unsqueeze(1) + koff                        # key index of the query itself
    win = pos - (window - 1) + torch.arange(window, device=q.device).unsqueeze(0)      # [S, window], oldest first
    win = torch.where(win < 0, torch.full_like(win, -1), win)
    comp = torch.where(cidx < 0, cidx, cidx + Tk)
    idx = torch.cat([win, comp], dim=1)
    pad = (-idx.shape[1]) % 128
    if pad:
        idx = F.pad(idx, (0, pad), value=-1)
    keys = torch.cat([kv, kvc], dim=0)
    out, teacher, _ = sparse_mla(q.contiguous(), keys, idx.to(torch.int32), scale, hd, sink)
    dist = teacher[:, window: window + k] / n_heads_total if want_dist else None
    return out, dist


def _chunk(q, kv, sink, kvc, cidx, s0: int, koff: int, qpos0: int, window: int, ratio: int, scale: float,
           n_heads_total: int, want_dist: bool):
    """q [Sc,H,hd] (local queries s0..s0+Sc), kv [Tk,hd] raw keys where local query s sits at key index s + koff,
    kvc [Tc,hd] | None compressed keys (global ids), cidx [Sc,k] compressed ids (-1 empty) | None; ``qpos0`` is the
    global position of local query 0."""
    Sc, H, hd = q.shape
    s1 = s0 + Sc
    t0 = max(0, s0 + koff - window + 1)
    kwin = kv[t0: s1 + koff]  # [W, hd]
    qh = q.transpose(0, 1)  # [H, Sc, hd]
    spos = torch.arange(s0, s1, device=q.device).unsqueeze(1)
    kpos = spos + koff
    tpos = torch.arange(t0, s1 + koff, device=q.device).unsqueeze(0)
    outside = (tpos > kpos) | (tpos <= kpos - window)  # [Sc, W]
    dense_ok = cidx is None or (kvc is not None and kvc.shape[0] <= DENSE_RATIO * cidx.shape[1])
    if _lib.on_device(q) and q.dtype in (torch.bfloat16, torch.float16) and dense_ok:
        # One GEMM over [window keys | compressed keys], one kernel for mask + sink + softmax, one GEMM back: the shared
        # KV latent is key and value at once, so the concatenated key block serves both products.
        from titan_b200.ops.masked_softmax import masked_softmax

        W = kwin.shape[0]
        blocks, masks, c_end = [kwin], [~outside], 0
        if kvc is not None and ratio > 1:
            if cidx is not None:
                c_end = kvc.shape[0]
                slot = torch.where(cidx < 0, c_end, cidx).long()  # empty slots point at a scratch column
                masks.append(torch.zeros(Sc, c_end + 1, dtype=torch.bool, device=q.device)
                             .scatter_(1, slot, True)[:, :c_end])
            else:
                c_end = min((qpos0 + s1) // ratio, kvc.shape[0])
                masks.append(torch.arange(c_end, device=q.device).unsqueeze(0) < (qpos0 + spos + 1) // ratio)
            blocks.append(kvc[:c_end])
        pad = (-(W + c_end)) % 8  # the kernel reads 16-byte vectors
        if pad:
            blocks.append(kv.new_zeros(pad, hd))
            masks.append(torch.zeros(Sc, pad, dtype=torch.bool, device=q.device))
        keys = torch.cat(blocks, dim=0) if len(blocks) > 1 else kwin
        allowed = torch.cat(masks, dim=1) if len(masks) > 1 else masks[0]
        p = masked_softmax(torch.matmul(qh * scale, keys.t()), allowed, 1.0, sink)  # [H, Sc, T]
        out = torch.matmul(p, keys).transpose(0, 1)
        if cidx is not None and c_end > 0 and want_dist:
            mass = p[..., W: W + c_end].detach().sum(0, dtype=torch.float32) / n_heads_total  # [Sc, Tc]
            return out, torch.gather(mass, 1, cidx.clamp(min=0).long())
        return (out,)
    logit_w = torch.matmul(qh, kwin.t()).float() * scale  # [H, Sc, W]
    logit_w = logit_w.masked_fill(outside.unsqueeze(0), float("-inf"))
    parts = [logit_w]
    ksel = None
    dense_sel = False
    if kvc is not None and ratio > 1:
        if cidx is not None and kvc.shape[0] <= DENSE_RATIO * cidx.shape[1]:
            # short compressed stream: all keys through one GEMM, the selection as a mask (no gather, no scatter-add)
            dense_sel = True
            c_end = kvc.shape[0]
            kc = kvc
            logit_c = torch.matmul(qh, kc.t()).float() * scale  # [H, Sc, Tc]
            slot = torch.where(cidx < 0, c_end, cidx).long()     # empty slots point at a scratch column
            allowed = torch.zeros(Sc, c_end + 1, dtype=torch.bool, device=q.device).scatter_(1, slot, True)[:, :c_end]
            logit_c = logit_c.masked_fill(~allowed.unsqueeze(0), float("-inf"))
        elif cidx is not None:
            ksel = gather_rows(kvc, cidx.clamp(min=0).long())  # [Sc, k, hd]
            logit_c = torch.einsum("hsd,skd->hsk", qh, ksel).float() * scale
            logit_c = logit_c.masked_fill((cidx < 0).unsqueeze(0), float("-inf"))
        else:
            c_end = min((qpos0 + s1) // ratio, kvc.shape[0])
            kc = kvc[:c_end]
            logit_c = torch.matmul(qh, kc.t()).float() * scale  # [H, Sc, c_end]
            hidden = torch.arange(c_end, device=q.device).unsqueeze(0) >= (qpos0 + spos + 1) // ratio
            logit_c = logit_c.masked_fill(hidden.unsqueeze(0), float("-inf"))
        parts.append(logit_c)
    parts.append(sink.float().view(H, 1, 1).expand(H, Sc, 1))
    p = torch.softmax(torch.cat(parts, dim=-1), dim=-1)
    W = logit_w.shape[-1]
    out = torch.matmul(p[..., :W].to(kv.dtype), kwin)  # [H, Sc, hd]
    dist = None
    if len(parts) == 3:
        pc = p[..., W:-1]
        if ksel is not None:
            out = out + torch.einsum("hsk,skd->hsd", pc.to(kv.dtype), ksel)
            if want_dist:
                dist = pc.detach().sum(0) / n_heads_total
        elif dense_sel:
            out = out + torch.matmul(pc.to(kv.dtype), kvc)
            if want_dist:  # head-mean probability at the selected keys, in the order of `cidx`
                mass = pc.detach().sum(0) / n_heads_total  # [Sc, Tc]
                dist = torch.gather(mass, 1, cidx.clamp(min=0).long())
        else:
            out = out + torch.matmul(pc.to(kv.dtype), kvc[: pc.shape[-1]])
    out = out.transpose(0, 1)
    return (out, dist) if dist is not None else (out,)


def smla_attention(q, kv, sink, kv_compress, compress_idx, window: int, ratio: int, scale: float,
                   want_dist: bool = False, *, n_heads_total: int | None = None, chunk: int | None = None,
                   q_pos0: int = 0, kv_pos0: int = 0, idx_offset: int | None = None):
    """q [B,S,H,hd], kv [B,Tk,hd], sink [H], kv_compress [B,Tc,hd] | None, compress_idx [B,S,k] | None (compressed ids
    + ``idx_offset``, default ``Tk`` as in the dense layout; -1 = empty) → (out [B,S,H,hd], dist [B,S,k] | None).

    Without context parallelism ``Tk == S``.  With it the local queries start at global position ``q_pos0`` and the raw
    keys at ``kv_pos0 <= q_pos0`` (the previous rank's window is prepended): ``Tk == S + q_pos0 - kv_pos0``; the
    compressed keys are global."""
    B, S, H, _ = q.shape
    n_heads_total = n_heads_total or H
    if chunk is None:
        # queries per chunk: as many as keep the fp32 logits of a chunk ([H, chunk, chunk + window + Tc]) near
        # 512 MB; few large chunks matter because this path is launch-bound on short sequences
        width = window + (kv_compress.shape[1] if kv_compress is not None else 0)
        chunk = 256
        while chunk < S and 4 * H * (2 * chunk) * (2 * chunk + width) <= (512 << 20):
            chunk *= 2
    koff = q_pos0 - kv_pos0
    if kv.shape[1] != S + koff:
        raise ValueError(f"raw keys must cover the local queries and their window: {kv.shape[1]} != {S} + {koff}")
    idx_offset = kv.shape[1] if idx_offset is None else idx_offset
    local_idx = None
    if compress_idx is not None:
        local_idx = torch.where(compress_idx < 0, compress_idx, compress_idx - idx_offset)
    outs, dists = [], []
    need_grad = torch.is_grad_enabled() and (q.requires_grad or kv.requires_grad)
    if _kernel_takes(q, kv_compress, compress_idx, window, ratio):
        for b in range(B):
            o, d = _smla_kernel_row(q[b], kv[b], sink, kv_compress[b], local_idx[b], koff, window, scale,
                                    n_heads_total, want_dist)
            outs.append(o)
            if d is not None:
                dists.append(d)
        out = torch.stack(outs)
        dist = torch.stack(dists).masked_fill(compress_idx < 0, 0.0) if dists else None
        return out, dist
    for b in range(B):
        ob, db = [], []
        for s0 in range(0, S, chunk):
            s1 = min(s0 + chunk, S)
            args = (q[b, s0:s1], kv[b], sink, None if kv_compress is None else kv_compress[b],
                    None if local_idx is None else local_idx[b, s0:s1], s0, koff, q_pos0, window, ratio, scale,
                    n_heads_total, want_dist)
            res = checkpoint(_chunk, *args, use_reentrant=False) if need_grad else _chunk(*args)
            ob.append(res[0])
            if len(res) > 1:
                db.append(res[1])
        outs.append(torch.cat(ob, dim=0))
        if db:
            dists.append(torch.cat(db, dim=0))
    out = torch.stack(outs)
    dist = torch.stack(dists).masked_fill(compress_idx < 0, 0.0) if dists else None
    return out, dist


def li_select(q_indexer, k_indexer, weights, ratio: int, index_topk: int, offset: int = 0, pos_offset: int = 0):
    """Fused counterpart of the eager selection: (idx [B,S,k] with ``offset`` added, -1 = empty; scores [B,S,k]).

    Selection (no gradient) runs on the scoring GEMM + radix-select kernels; the returned scores are recomputed at
    the selected keys only and carry the gradient to the indexer.  ``pos_offset`` is the global position of local
    query 0 (context parallelism: the keys are global, the queries a slice)."""
    from titan_b200.ops.dsa import _scoring_kernels_take, indexer_scores_from_selection, lightning_indexer_topk

    B = q_indexer.shape[0]
    k = min(index_topk, k_indexer.shape[1])
    idx, vals = lightning_indexer_topk(q_indexer.detach(), weights.detach(), k_indexer.detach().unsqueeze(2), k,
                                       pos_offset, ratio)
    idx = idx.long()
    safe = idx.clamp(min=0)
    T = k_indexer.shape[1]
    if _scoring_kernels_take(q_indexer) and T % 8 == 0:
        # forward values straight from the scoring kernel, fused backward (no [B,S,H,T] tensor in either direction)
        s = indexer_scores_from_selection(q_indexer, weights, k_indexer.unsqueeze(2), idx, vals)
        s = torch.where(idx < 0, torch.full_like(s, torch.finfo(q_indexer.dtype).min), s)
        return torch.where(idx < 0, idx, idx + offset), s
    if T <= DENSE_RATIO * k:
        # short key stream: score all keys with one GEMM per batch row and pick the selected ones (the gradient of a
        # gather along the key axis is a cheap scatter; no [B,S,k,D] tensor is built)
        dense = torch.einsum("bshd,btd->bsht", q_indexer, k_indexer)
        dense = (F.relu(dense) * weights.unsqueeze(-1)).sum(2)  # [B,S,T]
        s = torch.gather(dense, 2, safe)
    else:
        ksel = torch.stack([gather_rows(k_indexer[b], safe[b]) for b in range(B)])  # [B,S,k,D]
        s = torch.einsum("bshd,bskd->bshk", q_indexer, ksel)
        s = (F.relu(s) * weights.unsqueeze(-1)).sum(2)
    s = s.masked_fill(idx < 0, torch.finfo(q_indexer.dtype).min)
    return torch.where(idx < 0, idx, idx + offset), s
