"""DeepSeek-V4 building blocks (RoPE caches, index sets, eager sparse attention, Compressor, Indexer).

Model overview — DeepSeek-V4: hyper-connected residual streams, compressed-KV sparse attention, hash/sqrt-softplus MoE, MTP.

Per block (``x`` is ``[B, S, hc, D]``, ``hc`` parallel residual streams):

    y, post, comb = hc_pre(x)            # collapse streams → [B, S, D]  (mixing logits + Sinkhorn)
    y = attention(attention_norm(y))     # or moe(ffn_norm(y))
    x = hc_post(y, x, post, comb)        # write back into the hc streams

Attention is multi-query with ONE shared latent KV head of width ``head_dim`` (values = keys):

* queries: ``wq_a → RMSNorm → wq_b`` then a weight-free per-head RMS normalisation, RoPE on the last
  ``rope_head_dim`` dims;
* keys: ``wkv → RMSNorm`` + RoPE; every query sees its causal sliding window of ``window_size`` raw keys;
* layers with ``compress_ratio > 1`` also see compressed keys: the `Compressor` pools every ``ratio`` tokens into one
  key with a learned softmax gate (ratio 4 pools over two overlapping groups).  With ratio 4 a lightning `Indexer`
  (its own compressor + Hadamard rotation) picks the top-k compressed keys per query and is trained with the KL
  indexer loss; with ratio 128 all visible compressed keys are used;
* a learned per-head sink logit joins the softmax and is dropped afterwards;
* output: inverse RoPE on the value rope dims, grouped low-rank projection ``wo_a`` (per group) → ``wo_b``.

Parity: torchtitan_npu/models/deepseek_v4/model.py (Compressor :130-296, Indexer :298-364, LiLoss :366-457,
SparseAttention :553-624, LiCompute :626-657, Pre/Inner/PostAttention :659-897, block :1077-1207, HcHead :1209,
MTPModule :1253, DeepSeekV4Model :1341-1660) and models/deepseek_v4/moe.py.
"""

from __future__ import annotations

import math
import torch
import torch.nn as nn
import torch.nn.functional as F

from titan_b200.models.common.layers import Linear, RMSNorm
from titan_b200.models.common.rope import apply_rotary_emb_single_complex
from titan_b200.models.deepseek_v32.model import rotate_activation
from titan_b200.protocols.module import Module

__all__ = ["Compressor", "Indexer", "window_topk_idxs", "compress_visible_idxs", "li_compute",
           "sparse_attention_dense", "rope_tail", "precompute_v4_freqs"]


# --------------------------------------------------------------------------------------------------------------
# RoPE
# --------------------------------------------------------------------------------------------------------------
def precompute_v4_freqs(cfg: "V4Config", with_compressor: bool, device=None) -> torch.Tensor:
    """Complex cache ``[max_seq_len, rope_head_dim/2]``.  Layers with a compressor use ``compress_rope_theta`` with
    YaRN frequency interpolation; pure sliding-window layers use plain ``rope_theta``."""
    dim, base = cfg.rope_head_dim, (cfg.compress_rope_theta if with_compressor else cfg.rope_theta)
    freqs = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    orig = cfg.original_seq_len if with_compressor else 0
    if orig > 0:
        def corr_dim(rot):
            return dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(base))

        low, high = max(math.floor(corr_dim(cfg.beta_fast)), 0), min(math.ceil(corr_dim(cfg.beta_slow)), dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(dim // 2, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0, 1)
        smooth = 1 - ramp
        freqs = freqs / cfg.rope_factor * (1 - smooth) + freqs * smooth
    ang = torch.outer(torch.arange(cfg.max_seq_len, dtype=torch.float32, device=device), freqs)
    return torch.polar(torch.ones_like(ang), ang)


def rope_tail(x: torch.Tensor, freqs_cis: torch.Tensor, rd: int, positions=None, inverse: bool = False):
    """Rotate the last ``rd`` dims of ``x`` ([B,S,H,hd] or [B,S,hd]); the leading dims pass through."""
    squeeze = x.dim() == 3
    if squeeze:
        x = x.unsqueeze(2)
    rot = apply_rotary_emb_single_complex(x[..., -rd:], freqs_cis, positions, inverse=inverse)
    out = torch.cat([x[..., :-rd], rot], dim=-1)
    return out.squeeze(2) if squeeze else out


# --------------------------------------------------------------------------------------------------------------
# index sets
# --------------------------------------------------------------------------------------------------------------
def window_topk_idxs(window: int, seqlen: int, device=None) -> torch.Tensor:
    """[S, min(S, window)] raw-key indices of every query's causal window, -1 where the slot is in the future."""
    base = torch.arange(seqlen, device=device).unsqueeze(1)
    idx = (base - window + 1).clamp(min=0) + torch.arange(min(seqlen, window), device=device)
    return torch.where(idx > base, -1, idx)


def compress_visible_idxs(ratio: int, seqlen: int, offset: int = 0, device=None) -> torch.Tensor:
    """[S, S/ratio] all compressed keys a query may see (block c closes at token ``(c+1)·ratio - 1``), else -1."""
    m = torch.arange(seqlen // ratio, device=device).repeat(seqlen, 1)
    hidden = m >= (torch.arange(1, seqlen + 1, device=device).unsqueeze(1) // ratio)
    return torch.where(hidden, -1, m + offset)


def li_compute(q_indexer, k_indexer, weights, ratio: int, index_topk: int, offset: int = 0, pos_offset: int = 0):
    """Lightning-indexer selection over compressed keys.

    q_indexer [B,S,Hi,Di], k_indexer [B,Tc,Di], weights [B,S,Hi] → (idx [B,S,k] with ``offset`` added and -1
    for hidden keys, scores [B,S,k] – the selected logits, differentiable).  Local query ``s`` stands at global
    position ``pos_offset + s`` and sees the compressed keys whose block of ``ratio`` tokens is complete."""
    S, T = q_indexer.shape[1], k_indexer.shape[1]
    score = torch.einsum("bshd,btd->bsht", q_indexer, k_indexer)
    score = (F.relu(score) * weights.unsqueeze(-1)).sum(dim=2)
    base = torch.arange(S, device=score.device).unsqueeze(1) + pos_offset
    visible_end = (base + 1) // ratio
    hidden = torch.arange(T, device=score.device).unsqueeze(0) >= visible_end
    score = score + torch.where(hidden, torch.finfo(q_indexer.dtype).min, 0.0)
    vals, idx = score.topk(min(index_topk, T), dim=-1)
    return torch.where(idx >= visible_end, -1, idx + offset), vals


def sparse_attention_dense(q, kv, attn_sink, kv_compress, compress_idx, window: int, ratio: int, scale: float):
    """Eager oracle: dense logits over ``[raw keys | compressed keys | sink]`` with an index mask.

    q [B,S,H,hd], kv [B,S,hd], kv_compress [B,Tc,hd] | None, compress_idx [B,S,k] (already offset by S; -1 = empty)
    or None (= every visible compressed key).  Returns (out [B,S,H,hd], probs [B,H,S,S+Tc] fp32)."""
    B, S, H, _ = q.shape
    idx = window_topk_idxs(window, S, q.device).unsqueeze(0).expand(B, -1, -1)
    if ratio > 1 and kv_compress is not None:
        if compress_idx is None:
            compress_idx = compress_visible_idxs(ratio, S, S, q.device).unsqueeze(0).expand(B, -1, -1)
        idx = torch.cat([idx, compress_idx.to(idx.dtype)], dim=-1)
        kv = torch.cat([kv, kv_compress], dim=1)
    T = kv.shape[1]
    logits = torch.matmul(q.transpose(1, 2), kv.unsqueeze(1).transpose(2, 3)).float() * scale  # [B,H,S,T]
    idx = idx.masked_fill(idx < 0, T)  # empty slots point at a scratch column
    allowed = torch.zeros(B, 1, S, T + 1, dtype=torch.bool, device=q.device).scatter_(-1, idx.unsqueeze(1), True)
    logits = logits.masked_fill(~allowed[..., :T], float("-inf"))
    sink = attn_sink.float().view(1, H, 1, 1).expand(B, H, S, 1)
    probs = torch.softmax(torch.cat([logits, sink], dim=-1), dim=-1)[..., :T]
    out = torch.matmul(probs.to(kv.dtype), kv.unsqueeze(1))  # [B,H,S,hd]
    return out.transpose(1, 2).contiguous(), probs


# --------------------------------------------------------------------------------------------------------------
# Compressor / Indexer
# --------------------------------------------------------------------------------------------------------------
def _w(p):
    """Local view of a parameter that tensor parallelism keeps replicated (the computation is replicated too)."""
    return p.to_local() if hasattr(p, "to_local") else p


class Compressor(Module):
    """Pool every ``ratio`` tokens into one key: ``Σ_j softmax_j(gate_j + ape_j) · kv_j`` → RMSNorm → RoPE.

    With ratio 4 the projections are twice as wide: the first half of block ``c-1`` and the second half of block
    ``c`` are pooled together (``2·ratio`` candidates), so neighbouring compressed keys overlap.  The projections
    and the gate softmax run in fp32."""

    def __init__(self, cfg: "V4Config", ratio: int, head_dim: int):
        super().__init__()
        self.ratio, self.head_dim, self.rd = ratio, head_dim, cfg.rope_head_dim
        self.overlap = ratio == 4
        width = (2 if self.overlap else 1) * head_dim
        self.ape = nn.Parameter(torch.empty(ratio, width, dtype=torch.float32))
        self.wkv = Linear(cfg.dim, width, bias=False).to(torch.float32)
        self.wgate = Linear(cfg.dim, width, bias=False).to(torch.float32)
        self.norm = RMSNorm(head_dim, eps=cfg.norm_eps)

    def pool(self, kv: torch.Tensor, score: torch.Tensor) -> torch.Tensor:
        """kv, score [B, S, width] fp32 → pooled [B, S/ratio, head_dim] fp32 (one kernel on CUDA)."""
        from titan_b200.ops.compressor_pool import compressor_pool

        return compressor_pool(kv, score, _w(self.ape), self.ratio, self.head_dim, self.overlap)

    def forward(self, x: torch.Tensor, freqs_cis: torch.Tensor, positions=None,
                allow_residual: bool = False) -> torch.Tensor:
        B, S, _ = x.shape
        if S % self.ratio != 0:
            if not allow_residual:
                raise ValueError(f"sequence length {S} must be a multiple of the compression ratio {self.ratio}")
            # packed documents: the tokens after the last complete block stay uncompressed
            S = S // self.ratio * self.ratio
            x = x[:, :S]
            positions = positions[..., :S] if positions is not None else None
            if S == 0:
                return x.new_zeros(B, 0, self.head_dim)
        xf = x.float()
        kv = F.linear(xf, _w(self.wkv.weight).float())
        score = F.linear(xf, _w(self.wgate.weight).float())
        pooled = self.norm(self.pool(kv, score).to(x.dtype))
        if positions is not None:
            return rope_tail(pooled, freqs_cis, self.rd, positions[..., ::self.ratio])
        return rope_tail(pooled, freqs_cis[::self.ratio], self.rd)

    def init_states(self, *, init_std=0.02, **kw):
        nn.init.trunc_normal_(self.ape, mean=0.0, std=0.02)
        nn.init.trunc_normal_(self.wkv.weight, mean=0.0, std=0.02)
        nn.init.trunc_normal_(self.wgate.weight, mean=0.0, std=0.02)
        self.norm.init_states()


class Indexer(Module):
    """Lightning indexer over compressed keys: few-head queries from the q-LoRA latent, its own compressor for the
    keys, both Hadamard-rotated; per-head weights from the hidden state."""

    def __init__(self, cfg: "V4Config", ratio: int):
        super().__init__()
        self.n_heads, self.head_dim, self.rd = cfg.index_n_heads, cfg.index_head_dim, cfg.rope_head_dim
        self.wq_b = Linear(cfg.q_lora_rank, self.n_heads * self.head_dim, bias=False)
        self.weights_proj = Linear(cfg.dim, self.n_heads, bias=False)
        self.compressor = Compressor(cfg, ratio, self.head_dim)
        self.scale = self.head_dim ** -0.5 * self.n_heads ** -0.5

    def forward(self, x, qr, freqs_cis, positions=None, allow_residual: bool = False):
        B, S, _ = x.shape
        q = self.wq_b(qr).view(B, S, self.n_heads, self.head_dim)
        q = rotate_activation(rope_tail(q, freqs_cis, self.rd, positions))
        k = rotate_activation(self.compressor(x, freqs_cis, positions, allow_residual))
        return q, k, self.weights_proj(x) * self.scale

    def init_states(self, *, init_std=0.02, **kw):
        nn.init.trunc_normal_(self.wq_b.weight, mean=0.0, std=0.02)
        nn.init.trunc_normal_(self.weights_proj.weight, mean=0.0, std=0.02)
        self.compressor.init_states(init_std=init_std)
