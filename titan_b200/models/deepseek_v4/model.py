"""DeepSeek-V4 attention (pre / inner / post), MoE wrapper and the stream-collapsing head.

Module names follow the reference so checkpoints map one to one:
``layers.N.attention.{pre_attention,inner_attention,post_attention}``, ``layers.N.moe``, ``layers.N.hc_*``,
``layers.<last>.hc_head``; MTP modules are appended to ``layers`` with ids ``n_layers ..``.

Parity: torchtitan_npu/models/deepseek_v4/model.py:659-1660.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from titan_b200.models.common.dsa_indexer_loss import (
    DSAIndexerLossAutoScaler,
    DSAIndexerLossLoggingHelper,
    dsa_indexer_loss,
)
from titan_b200.models.common.layers import Linear, RMSNorm
from titan_b200.models.common.moe import MoE, MoEArgs
from titan_b200.models.deepseek_v4.layers import (
    Compressor,
    Indexer,
    li_compute,
    rope_tail,
    sparse_attention_dense,
)
from titan_b200.ops import mhc
from titan_b200.protocols.module import Module

__all__ = ["PreAttention", "InnerAttention", "PostAttention", "V4Attention", "HcHead", "V4MoE"]


def _ratio_of(cfg, layer_id: int) -> int:
    return cfg.compress_ratios[layer_id] if layer_id < cfg.n_layers else cfg.mtp_layer_compress_ratio


class PreAttention(Module):
    """Projections in front of the attention core: queries, the shared KV latent, compressed KV, indexer inputs."""

    def __init__(self, layer_id: int, cfg: "V4Config"):
        super().__init__()
        self.n_heads, self.head_dim, self.rd, self.eps = cfg.n_heads, cfg.head_dim, cfg.rope_head_dim, cfg.norm_eps
        self.compress_ratio = _ratio_of(cfg, layer_id)
        self.wq_a = Linear(cfg.dim, cfg.q_lora_rank, bias=False)
        self.q_norm = RMSNorm(cfg.q_lora_rank, eps=cfg.norm_eps)
        self.wq_b = Linear(cfg.q_lora_rank, cfg.n_heads * cfg.head_dim, bias=False)
        self.wkv = Linear(cfg.dim, cfg.head_dim, bias=False)
        self.kv_norm = RMSNorm(cfg.head_dim, eps=cfg.norm_eps)
        if self.compress_ratio == 4:
            self.compressor = Compressor(cfg, 4, cfg.head_dim)
            self.indexer = Indexer(cfg, 4)
        elif self.compress_ratio > 1:
            self.compressor_128 = Compressor(cfg, self.compress_ratio, cfg.head_dim)

    def forward(self, x, freqs_cis, positions=None, allow_residual: bool = False):
        """``allow_residual``: packed documents whose length is no multiple of the compression ratio keep their tail
        uncompressed instead of raising."""
        B, S, _ = x.shape
        qr = self.q_norm(self.wq_a(x))
        q = self.wq_b(qr).unflatten(-1, (-1, self.head_dim))  # local heads under tensor parallelism
        q = q * torch.rsqrt(q.float().square().mean(-1, keepdim=True) + self.eps).to(q.dtype)
        q = rope_tail(q, freqs_cis, self.rd, positions)
        kv = rope_tail(self.kv_norm(self.wkv(x)), freqs_cis, self.rd, positions)
        kv_compress = q_idx = k_idx = weights = None
        if self.compress_ratio == 4:
            # the indexer learns from its own KL loss only: its inputs are cut from the main graph
            q_idx, k_idx, weights = self.indexer(x.detach(), qr.detach(), freqs_cis, positions, allow_residual)
            kv_compress = self.compressor(x, freqs_cis, positions, allow_residual)
        elif self.compress_ratio > 1:
            kv_compress = self.compressor_128(x, freqs_cis, positions, allow_residual)
        return q, kv, kv_compress, q_idx, k_idx, weights

    def init_states(self, *, init_std=0.02, **kw):
        for lin in (self.wq_a, self.wq_b, self.wkv):
            nn.init.trunc_normal_(lin.weight, mean=0.0, std=0.02)
        for n in (self.q_norm, self.kv_norm):
            nn.init.trunc_normal_(n.weight, mean=1.0, std=0.02)
        for name in ("compressor", "compressor_128", "indexer"):
            if hasattr(self, name):
                getattr(self, name).init_states(init_std=init_std)


class InnerAttention(Module):
    """The attention core: index selection, sparse attention with sink, indexer loss.

    ``self.core`` is the swap point of the ``b200_smla`` converter: a callable
    ``(q, kv, attn_sink, kv_compress, compress_idx, window, ratio, scale, want_dist) → (out, dist)`` where ``dist``
    is the head-mean probability on the selected compressed keys ``[B, S, k]`` (or None)."""

    def __init__(self, layer_id: int, cfg: "V4Config"):
        super().__init__()
        self.layer_id, self.n_layers_total = layer_id, cfg.n_layers + cfg.num_mtp_modules
        self.n_heads = cfg.n_heads
        self.compress_ratio = _ratio_of(cfg, layer_id)
        self.window, self.index_topk = cfg.window_size, cfg.index_topk
        self.scale = cfg.head_dim ** -0.5
        self.enable_indexer_loss = cfg.enable_indexer_loss
        self.attn_sink = nn.Parameter(torch.empty(cfg.n_heads, dtype=torch.float32))
        self.core = None
        self.tp_group = None  # set by the tensor-parallel plan: heads are split over this group
        self.select = None  # optional fused selection: (q_idx, k_idx, weights, ratio, topk, offset) → (idx, vals)

    def _dense_core(self, q, kv, sink, kv_compress, compress_idx, want_dist):
        S = q.shape[1]
        out, probs = sparse_attention_dense(q, kv, sink, kv_compress, compress_idx, self.window,
                                            self.compress_ratio, self.scale)
        dist = None
        if want_dist:
            cmp = probs[..., S:].detach().sum(dim=1) / self.n_heads  # [B,S,Tc]
            local = (compress_idx - S).clamp(min=0)
            dist = torch.gather(cmp, -1, local).masked_fill(compress_idx < 0, 0.0)
        return out, dist

    def forward(self, q, kv, kv_compress, q_idx, k_idx, weights, q_pos0: int = 0, kv_pos0: int = 0):
        """``q_pos0`` / ``kv_pos0``: global positions of the first local query / raw key (context parallelism hands in
        a slice of the queries with the previous rank's window prepended to the keys; compressed keys are global)."""
        offset = kv.shape[1]
        sink = self.attn_sink.to_local() if hasattr(self.attn_sink, "to_local") else self.attn_sink
        compress_idx = scores = None
        has_li = q_idx is not None
        if has_li:
            sel = self.select or li_compute
            compress_idx, scores = sel(q_idx, k_idx, weights, self.compress_ratio, self.index_topk, offset, q_pos0)
        want = has_li and self.enable_indexer_loss and torch.is_grad_enabled()
        if self.core is not None:
            out, dist = self.core(q, kv, sink, kv_compress, compress_idx, self.window, self.compress_ratio,
                                  self.scale, want, q_pos0=q_pos0, kv_pos0=kv_pos0)
        else:
            if q_pos0 or kv_pos0:
                raise NotImplementedError("the dense attention oracle has no context-parallel form")
            out, dist = self._dense_core(q, kv, sink, kv_compress, compress_idx, want)
        if want:
            if self.tp_group is not None:  # every rank holds the probability mass of its own heads only
                import torch.distributed as c10d

                dist = dist.contiguous()
                c10d.all_reduce(dist, group=self.tp_group)
            loss = dsa_indexer_loss(dist, scores, self.scale, eps=1e-10)
            DSAIndexerLossLoggingHelper.save_loss_to_tracker(loss, self.layer_id, self.n_layers_total)
            out = DSAIndexerLossAutoScaler.apply(out, loss)
        return out

    def init_states(self, **kw):
        nn.init.trunc_normal_(self.attn_sink, mean=0.0, std=0.02)


class PostAttention(Module):
    """Inverse RoPE on the value rope dims, then the grouped low-rank output projection."""

    def __init__(self, cfg: "V4Config"):
        super().__init__()
        self.n_heads, self.head_dim, self.rd = cfg.n_heads, cfg.head_dim, cfg.rope_head_dim
        self.n_groups, self.o_lora_rank = cfg.o_groups, cfg.o_lora_rank
        self.wo_a = Linear(cfg.n_heads * cfg.head_dim // cfg.o_groups, cfg.o_groups * cfg.o_lora_rank, bias=False)
        self.wo_b = Linear(cfg.o_groups * cfg.o_lora_rank, cfg.dim, bias=False)

    def forward(self, o, freqs_cis, positions=None):
        B, S, H, _ = o.shape
        groups = self.n_groups // (self.n_heads // H)  # local groups under tensor parallelism
        o = rope_tail(o, freqs_cis, self.rd, positions, inverse=True).reshape(B, S, groups, -1)
        w = self.wo_a.weight
        w = w.to_local() if hasattr(w, "to_local") else w
        o = torch.einsum("bsgd,grd->bsgr", o, w.view(groups, self.o_lora_rank, -1))
        return self.wo_b(o.reshape(B, S, -1))

    def init_states(self, **kw):
        nn.init.trunc_normal_(self.wo_a.weight, mean=0.0, std=0.02)
        nn.init.trunc_normal_(self.wo_b.weight, mean=0.0, std=0.02)


class V4Attention(Module):
    def __init__(self, layer_id: int, cfg: "V4Config"):
        super().__init__()
        self.pre_attention = PreAttention(layer_id, cfg)
        self.inner_attention = InnerAttention(layer_id, cfg)
        self.post_attention = PostAttention(cfg)

    def forward(self, x, freqs_cis, attention_masks=None, positions=None):
        if getattr(self, "cp", None) is not None:  # context parallelism: set by its strategy
            return self.cp.forward(self, x, freqs_cis)
        ranges = getattr(attention_masks, "doc_ranges", None)
        if ranges is not None:
            # packed stream [1, T, D]: window, compressor, indexer and attention see one document at a time (its
            # positions restart at 0, so no explicit positions are needed inside a document)
            if x.shape[0] != 1:
                raise ValueError("a packed DeepSeek-V4 stream has batch size 1")
            return torch.cat([self._one_sequence(x[:, a:b], freqs_cis, None, True) for a, b in ranges], dim=1)
        return self._one_sequence(x, freqs_cis, positions, False)

    def _one_sequence(self, x, freqs_cis, positions, allow_residual: bool):
        q, kv, kv_c, q_idx, k_idx, w = self.pre_attention(x, freqs_cis, positions, allow_residual)
        if kv_c is not None and kv_c.shape[1] == 0:  # shorter than one block: window attention only
            kv_c = q_idx = k_idx = w = None
        o = self.inner_attention(q, kv, kv_c, q_idx, k_idx, w)
        return self.post_attention(o, freqs_cis, positions)

    def init_states(self, *, init_std=0.02, **kw):
        self.pre_attention.init_states(init_std=init_std)
        self.inner_attention.init_states()
        self.post_attention.init_states()


class V4MoE(MoE):
    """Common MoE with the V4 specifics: SwiGLU clamp also on the shared expert; hash-routed layers carry no
    load-balancing bias."""

    def __init__(self, dim, hidden_dim, args: MoEArgs, *, layer_id: int, vocab_size: int):
        super().__init__(dim, hidden_dim, args, layer_id=layer_id, vocab_size=vocab_size)
        if self.shared_experts is not None:
            self.shared_experts.swiglu_limit = args.swiglu_limit
        self.hash_routed = layer_id < args.n_hash_layers
        if self.hash_routed and self.load_balance_coeff is not None:
            del self.expert_bias
            self.expert_bias = None
            self.load_balance_coeff = None


class HcHead(Module):
    def __init__(self, cfg: "V4Config"):
        super().__init__()
        self.norm_eps, self.hc_eps = cfg.norm_eps, cfg.hc_eps
        self.hc_head_fn = nn.Parameter(torch.empty(cfg.hc_mult, cfg.hc_mult * cfg.dim, dtype=torch.float32))
        self.hc_head_base = nn.Parameter(torch.empty(cfg.hc_mult, dtype=torch.float32))
        self.hc_head_scale = nn.Parameter(torch.empty(1, dtype=torch.float32))

    def forward(self, x):
        return mhc.hc_head(x, self.hc_head_fn, self.hc_head_scale, self.hc_head_base, self.hc_eps, self.norm_eps)

    def init_states(self, **kw):
        for p in (self.hc_head_fn, self.hc_head_base, self.hc_head_scale):
            nn.init.trunc_normal_(p, mean=0.0, std=0.02)
