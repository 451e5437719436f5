"""DeepSeek-V3.2: MLA in absorb mode + lightning-indexer sparse attention (DSA) + MTP modules.

Attention runs in three stages so kernels, context parallelism and loss hooks attach at clean seams:

* `PreAttention`  – q-LoRA (``wq_a → q_norm → wq_b``), KV latent (``wkv_a → kv_norm``), RoPE; in absorb mode
  ``q_nope`` is multiplied by ``W_uk`` so keys and values are ONE shared latent head of width
  ``kv_lora_rank (+ rope)``; the `Indexer` (64 heads × 128, LayerNorm on k, non-interleaved RoPE, Hadamard
  rotation, fp32 head weights) runs on detached inputs.
* `DSASparseAttention` (``inner_attention``) – eager oracle: index scores
  ``Σ_h w[s,h]·relu(q_idx[s,h]·k_idx[t])`` → causal mask → top-k keys per query → masked softmax attention →
  KL indexer loss against the head-summed main attention mass on the selected keys.  The `b200_dsa`
  converter swaps this for the fused kernels.
* `PostAttention` – ``W_uv`` un-absorb, ``wo``, loss auto-scaler + logging.

Blocks carry the residual; `MTPModule`s after the main layers predict further tokens (the model then
returns a list of logits).

Parity: torchtitan_npu/models/deepseek_v32/model.py:41-776.  FQNs follow the reference's adapter map
(models/deepseek_v32/state_dict_adapter.py:81-120): ``layers.N.attention.pre_attention.{wq_a,q_norm,wq_b,wkv_a,
kv_norm,wkv_b,indexer.{wq_b,wk,k_norm,weights_proj}}`` and ``layers.N.attention.post_attention.wo``; MTP depth i
lives under ``mtp_layers.i`` and is exported to HF as layer ``n_layers + i``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from titan_b200.models.common.dsa_indexer_loss import (
    DSAIndexerLoss,
    DSAIndexerLossAutoScaler,
    DSAIndexerLossLoggingHelper,
)
from titan_b200.models.common.layers import Embedding, FeedForward, LayerNorm, Linear, RMSNorm
from titan_b200.models.common.moe import MoE, MoEArgs
from titan_b200.models.common.rope import (
    apply_rotary_emb_single_complex,
    precompute_freqs_cis,
    yarn_inv_freq,
)
from titan_b200.protocols.module import BaseModelConfig, Module, ModuleDict

__all__ = ["DeepSeekV32Model", "Indexer", "DSASparseAttention", "PreAttention", "PostAttention", "V32Attention",
           "MTPModule", "hadamard_transform", "rotate_activation", "index_scores", "apply_rope_half"]


def hadamard_transform(x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Fast Walsh–Hadamard transform over the last dim (zero-padded to a power of two)."""
    shape = x.shape
    n = shape[-1]
    m = 1 << (n - 1).bit_length()
    out = F.pad(x.reshape(-1, n), (0, m - n)) if m != n else x.reshape(-1, n)
    h = 1
    while h < m:
        out = out.view(-1, m // (2 * h), 2, h)
        a, b = out[:, :, 0, :], out[:, :, 1, :]
        out = torch.stack((a + b, a - b), dim=2).reshape(-1, m)
        h *= 2
    return (out[..., :n] * scale).reshape(shape)


def rotate_activation(x: torch.Tensor) -> torch.Tensor:
    if (x.is_cuda or x.is_meta) and x.dtype in (torch.bfloat16, torch.float16) and x.size(-1) in (64, 128, 256, 512):
        from titan_b200.ops.hadamard import hadamard

        return hadamard(x)  # FWHT kernel: one warp per row, butterflies in registers + shuffles
    return hadamard_transform(x, scale=x.size(-1) ** -0.5)


def apply_rope_half(x: torch.Tensor, freqs_cis: torch.Tensor, positions=None) -> torch.Tensor:
    """Non-interleaved (half-rotate) RoPE driven by the complex cache: pairs are (x[i], x[i + D/2])."""
    d = x.shape[-1]
    inter = torch.stack((x[..., : d // 2], x[..., d // 2:]), dim=-1).flatten(-2)
    y = apply_rotary_emb_single_complex(inter, freqs_cis, positions)
    y = y.view(*y.shape[:-1], d // 2, 2)
    return torch.cat((y[..., 0], y[..., 1]), dim=-1)


def index_scores(q: torch.Tensor, weights: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
    """q [B,S,H,D], weights [B,S,H], k [B,T,1,D] → scores [B,S,T] = Σ_h w·relu(q·k) in fp32."""
    p = torch.matmul(q.float().transpose(1, 2), k.float().permute(0, 2, 3, 1))  # [B,H,S,T]
    return (F.relu(p) * weights.float().permute(0, 2, 1).unsqueeze(-1)).sum(dim=1)


class Indexer(Module):
    def __init__(self, cfg: "DeepSeekV32Model.Config"):
        super().__init__()
        self.n_heads, self.head_dim = cfg.index_n_heads, cfg.index_head_dim
        self.rope_head_dim, self.index_topk = cfg.qk_rope_head_dim, cfg.index_topk
        self.wq_b = Linear(cfg.q_lora_rank, self.n_heads * self.head_dim)
        self.wk = Linear(cfg.dim, self.head_dim)
        self.k_norm = LayerNorm(self.head_dim)
        self.weights_proj = Linear(cfg.dim, self.n_heads, dtype=torch.float32)  # kept in fp32
        self.softmax_scale = self.head_dim ** -0.5

    def forward(self, x, qr, freqs_cis, positions=None):
        bsz, seqlen, _ = x.shape
        q = self.wq_b(qr).view(bsz, seqlen, self.n_heads, self.head_dim)
        q_pe, q_nope = torch.split(q, [self.rope_head_dim, self.head_dim - self.rope_head_dim], dim=-1)
        q = torch.cat([apply_rope_half(q_pe, freqs_cis, positions), q_nope], dim=-1)
        k = self.k_norm(self.wk(x))
        k_pe, k_nope = torch.split(k, [self.rope_head_dim, self.head_dim - self.rope_head_dim], dim=-1)
        k_pe = apply_rope_half(k_pe.unsqueeze(2), freqs_cis, positions).squeeze(2)
        k = torch.cat([k_pe, k_nope], dim=-1).unsqueeze(2)
        q, k = rotate_activation(q), rotate_activation(k)
        weights = self.weights_proj(x.float()) * (self.n_heads ** -0.5) * self.softmax_scale
        return q, weights, k

    def init_states(self, *, init_std=0.02, **kw):
        self.wq_b.init_states(init_std=init_std)
        self.wk.init_states(init_std=init_std)
        self.weights_proj.init_states(init_std=init_std)
        self.k_norm.init_states()


class DSASparseAttention(Module):
    """Eager oracle of index → top-k → sparse attention → indexer loss (the spec the fused path is tested against)."""

    def __init__(self):
        super().__init__()
        self.compute_dsa_indexer_loss = DSAIndexerLoss()

    def forward(self, q, k, v, attn_mask=None, scale=None, q_indexer=None, k_indexer=None, weights=None,
                index_topk: int | None = None):
        """q [B,H,S,Dq], k [B,Hk,T,Dq], v [B,Hk,T,Dv] with Hk ∈ {1, H} → (loss, out [B,H,S,Dv])."""
        bsz = q.size(0)
        if q_indexer is None:
            out = F.scaled_dot_product_attention(q, k.expand(-1, q.shape[1], -1, -1), v.expand(-1, q.shape[1], -1, -1),
                                                 attn_mask=attn_mask, scale=scale, is_causal=attn_mask is None)
            return q.new_zeros(1), out
        score = index_scores(q_indexer, weights, k_indexer)  # [B, S, T]
        seqlen, kvlen = score.shape[1], score.shape[2]
        if attn_mask is None:
            # query s (global position offset + s) may see keys t <= its position; with CP the query block is the
            # tail of the gathered key range
            offset = kvlen - seqlen
            pos_q = torch.arange(seqlen, device=q.device).unsqueeze(-1) + offset
            future = torch.arange(kvlen, device=q.device).unsqueeze(0) > pos_q
            attn_mask = torch.zeros(bsz, seqlen, kvlen, device=q.device).masked_fill(future, float("-inf"))
        else:
            offset = kvlen - seqlen
            pos_q = torch.arange(seqlen, device=q.device).unsqueeze(-1) + offset
        score = score + attn_mask
        kk = min(index_topk or kvlen, kvlen)
        topk_score, topk_idx = score.topk(kk, dim=-1)
        valid = topk_idx <= pos_q.unsqueeze(0)
        topk_idx = torch.where(valid, topk_idx, torch.full_like(topk_idx, kvlen - 1))
        index_mask = torch.full((bsz, seqlen, kvlen), float("-inf"), device=q.device).scatter_(-1, topk_idx, 0.0)
        masked = attn_mask + index_mask
        masked = (torch.isinf(masked) & (masked < 0)).unsqueeze(1)  # True = masked out
        h = q.shape[1]
        out = F.scaled_dot_product_attention(q, k.expand(-1, h, -1, -1), v.expand(-1, h, -1, -1), attn_mask=~masked,
                                             scale=scale, is_causal=False)
        # teacher: head-summed main attention on the selected keys (no gradient into the main model)
        attn = (q.detach() @ k.detach().transpose(-1, -2)) * (scale if scale is not None else q.shape[-1] ** -0.5)
        attn = attn.masked_fill(masked, float("-inf"))
        attn = torch.nan_to_num(F.softmax(attn, dim=-1, dtype=torch.float32)).sum(dim=1)
        sel = torch.gather(attn, -1, topk_idx).masked_fill(~valid, 0.0)
        loss = self.compute_dsa_indexer_loss(sel, topk_score, topk_idx, 1.0)
        return loss, out


class PreAttention(Module):
    def __init__(self, cfg: "DeepSeekV32Model.Config"):
        super().__init__()
        self.n_heads = cfg.n_heads
        self.q_lora_rank, self.kv_lora_rank = cfg.q_lora_rank, cfg.kv_lora_rank
        self.qk_nope, self.qk_rope, self.v_head_dim = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.qk_head_dim = self.qk_nope + self.qk_rope
        self.enable_mla_absorb = cfg.enable_mla_absorb
        self.wq_a = Linear(cfg.dim, self.q_lora_rank)
        self.q_norm = RMSNorm(self.q_lora_rank, eps=cfg.norm_eps)
        self.wq_b = Linear(self.q_lora_rank, self.n_heads * self.qk_head_dim)
        self.wkv_a = Linear(cfg.dim, self.kv_lora_rank + self.qk_rope)
        self.kv_norm = RMSNorm(self.kv_lora_rank, eps=cfg.norm_eps)
        self.wkv_b = Linear(self.kv_lora_rank, self.n_heads * (self.qk_nope + self.v_head_dim))
        self.indexer = Indexer(cfg)
        self.softmax_scale = self.qk_head_dim ** -0.5
        if cfg.max_seq_len > cfg.original_seq_len:
            m = 0.1 * cfg.mscale * math.log(cfg.rope_factor) + 1.0
            self.softmax_scale *= m * m

    def forward(self, x, freqs_cis, attention_masks=None, positions=None):
        bsz, seqlen, _ = x.shape
        qr = self.q_norm(self.wq_a(x))
        q = self.wq_b(qr).view(bsz, seqlen, -1, self.qk_head_dim)
        q_nope, q_pe = torch.split(q, [self.qk_nope, self.qk_rope], dim=-1)
        q_pe = apply_rotary_emb_single_complex(q_pe, freqs_cis, positions)
        kv, k_pe = torch.split(self.wkv_a(x), [self.kv_lora_rank, self.qk_rope], dim=-1)
        k_pe = apply_rotary_emb_single_complex(k_pe.unsqueeze(2), freqs_cis, positions)
        w_uv_t = None
        if self.enable_mla_absorb:
            kv = self.kv_norm(kv)
            w = self.wkv_b.weight
            w = w.to_local() if hasattr(w, "to_local") else w
            w = w.reshape(-1, self.qk_nope + self.v_head_dim, self.kv_lora_rank)
            w_uk, w_uv = w[:, : self.qk_nope], w[:, self.qk_nope:]
            w_uv_t = w_uv.permute(0, 2, 1).contiguous()
            q_nope = torch.einsum("bshq,hqr->bshr", q_nope, w_uk.to(q_nope.dtype))
            k = torch.cat([kv.unsqueeze(2), k_pe], dim=-1)  # one shared latent head
            v = kv.unsqueeze(2)
        else:
            kvb = self.wkv_b(self.kv_norm(kv)).view(bsz, seqlen, -1, self.qk_nope + self.v_head_dim)
            k_nope, v = torch.split(kvb, [self.qk_nope, self.v_head_dim], dim=-1)
            k = torch.cat([k_nope, k_pe.expand(-1, -1, k_nope.shape[2], -1)], dim=-1)
        q = torch.cat([q_nope, q_pe], dim=-1)
        q_idx, weights, k_idx = self.indexer(x.detach(), qr.detach(), freqs_cis, positions)
        return (q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attention_masks, self.softmax_scale, q_idx,
                k_idx, weights, self.indexer.index_topk, w_uv_t)

    def init_states(self, *, init_std=0.02, **kw):
        for lin in (self.wq_a, self.wq_b, self.wkv_a, self.wkv_b):
            lin.init_states(init_std=0.02)
        self.q_norm.init_states()
        self.kv_norm.init_states()
        self.indexer.init_states(init_std=init_std)


class PostAttention(Module):
    def __init__(self, cfg: "DeepSeekV32Model.Config", num_total_layers: int):
        super().__init__()
        self.enable_mla_absorb = cfg.enable_mla_absorb
        self.wo = Linear(cfg.n_heads * cfg.v_head_dim, cfg.dim)
        self.n_layers = num_total_layers

    def forward(self, x, output, w_uv_t, loss, layer_id):
        bsz, seqlen, _ = x.shape
        if self.enable_mla_absorb and w_uv_t is not None:
            output = torch.einsum("bhsr,hrv->bhsv", output, w_uv_t.to(output.dtype))
        output = self.wo(output.transpose(1, 2).contiguous().view(bsz, seqlen, -1))
        DSAIndexerLossLoggingHelper.save_loss_to_tracker(loss, layer_id, self.n_layers)
        return DSAIndexerLossAutoScaler.apply(output, loss)

    def init_states(self, *, init_std=0.02, **kw):
        self.wo.init_states(init_std=init_std)


class V32Attention(Module):
    def __init__(self, cfg: "DeepSeekV32Model.Config", num_total_layers: int):
        super().__init__()
        self.pre_attention = PreAttention(cfg)
        self.inner_attention = DSASparseAttention()
        self.post_attention = PostAttention(cfg, num_total_layers)

    # checkpoint FQNs stay flat (layers.N.attention.wq_a …): expose the stage parameters under this module
    def forward(self, x, freqs_cis, attention_masks=None, positions=None, layer_id: int | None = None):
        q, k, v, mask, scale, q_idx, k_idx, w, topk, w_uv_t = self.pre_attention(x, freqs_cis, attention_masks,
                                                                                  positions)
        loss, out = self.inner_attention(q, k, v, attn_mask=mask, scale=scale, q_indexer=q_idx, k_indexer=k_idx,
                                         weights=w, index_topk=topk)
        return self.post_attention(x, out, w_uv_t, loss, layer_id)

    def init_states(self, *, init_std=0.02, **kw):
        self.pre_attention.init_states(init_std=init_std)
        self.post_attention.init_states(init_std=init_std)


class V32Block(Module):
    def __init__(self, layer_id: int, cfg: "DeepSeekV32Model.Config", num_total_layers: int, moe: bool | None = None):
        super().__init__()
        self.layer_id = layer_id
        self.attention = V32Attention(cfg, num_total_layers)
        self.attention_norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.ffn_norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.moe_enabled = (layer_id >= cfg.n_dense_layers) if moe is None else moe
        if self.moe_enabled:
            self.moe = MoE(cfg.dim, cfg.moe_inter_dim, cfg.moe_args, layer_id=layer_id, vocab_size=cfg.vocab_size)
        else:
            self.feed_forward = FeedForward(dim=cfg.dim, hidden_dim=cfg.inter_dim)
        self.weight_init_std = 0.02 / (2 * (layer_id + 1)) ** 0.5

    def forward(self, x, freqs_cis, attention_masks=None, positions=None):
        x = x + self.attention(self.attention_norm(x), freqs_cis, attention_masks, positions, self.layer_id)
        h = self.ffn_norm(x)
        return x + (self.moe(h) if self.moe_enabled else self.feed_forward(h))

    def init_states(self, *, buffer_device=None, **kw):
        self.attention_norm.init_states()
        self.ffn_norm.init_states()
        self.attention.init_states(init_std=self.weight_init_std)
        if self.moe_enabled:
            self.moe.init_states(init_std=self.weight_init_std, buffer_device=buffer_device)
        else:
            self.feed_forward.init_states(init_std=self.weight_init_std)


class MTPModule(Module):
    """Multi-token prediction depth k: fuse the previous hidden state with the embedding of the next token."""

    def __init__(self, layer_id: int, cfg: "DeepSeekV32Model.Config", num_total_layers: int):
        super().__init__()
        self.enorm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.hnorm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.eh_proj = Linear(2 * cfg.dim, cfg.dim)
        self.block = V32Block(layer_id, cfg, num_total_layers, moe=True)
        self.norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)

    def forward(self, h_prev, emb_next, freqs_cis, attention_masks=None, positions=None):
        h = self.eh_proj(torch.cat([self.enorm(emb_next), self.hnorm(h_prev)], dim=-1))
        h = self.block(h, freqs_cis, attention_masks, positions)
        return h, self.norm(h)

    def init_states(self, *, buffer_device=None, **kw):
        for n in (self.enorm, self.hnorm, self.norm):
            n.init_states()
        self.eh_proj.init_states()
        self.block.init_states(buffer_device=buffer_device)


class DeepSeekV32Model(Module):
    @dataclass(kw_only=True)
    class Config(BaseModelConfig):
        dim: int = 2048
        inter_dim: int = 10944
        moe_inter_dim: int = 1408
        n_layers: int = 12
        n_dense_layers: int = 1
        n_heads: int = 16
        vocab_size: int = 102400
        norm_eps: float = 1e-6
        moe_args: MoEArgs = field(default_factory=MoEArgs)
        q_lora_rank: int = 1536
        kv_lora_rank: int = 512
        qk_nope_head_dim: int = 128
        qk_rope_head_dim: int = 64
        v_head_dim: int = 128
        index_n_heads: int = 64
        index_head_dim: int = 128
        index_topk: int = 2048
        enable_mla_absorb: bool = True
        num_mtp_modules: int = 0
        max_seq_len: int = 4096
        original_seq_len: int = 4096
        rope_theta: float = 10000.0
        rope_factor: float = 40
        beta_fast: int = 32
        beta_slow: int = 1
        mscale: float = 1.0
        use_grouped_mm: bool = True

        def update_from_config(self, *, trainer_config, **kw) -> None:
            self.max_seq_len = trainer_config.training.seq_len + trainer_config.training.num_mtp_modules
            self.num_mtp_modules = trainer_config.training.num_mtp_modules
            self.moe_args._debug_force_load_balance = trainer_config.debug.moe_force_load_balance

        def get_nparams_and_flops(self, model, seq_len):
            nparams = emb = routed = 0
            for name, p in model.named_parameters():
                nparams += p.numel()
                if "tok_embeddings" in name:
                    emb += p.numel()
                elif ".moe.experts." in name:
                    routed += p.numel()
            active = nparams - emb - routed + routed * self.moe_args.top_k // max(self.moe_args.num_experts, 1)
            k_eff = min(self.index_topk, seq_len)
            attn = 12 * self.n_layers * self.n_heads * (self.kv_lora_rank + self.qk_rope_head_dim) * k_eff // 2
            idx = 6 * self.n_layers * self.index_n_heads * self.index_head_dim * seq_len // 2
            return nparams, 6 * active + attn + idx

    def __init__(self, cfg: "DeepSeekV32Model.Config"):
        super().__init__()
        self.config = cfg
        self.n_layers = cfg.n_layers
        total = cfg.n_layers + cfg.num_mtp_modules
        self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim)
        self.register_buffer("freqs_cis", self._precompute(), persistent=False)
        self.layers = ModuleDict({str(i): V32Block(i, cfg, total) for i in range(cfg.n_layers)})
        self.mtp_layers = ModuleDict({str(i): MTPModule(cfg.n_layers + i, cfg, total)
                                      for i in range(cfg.num_mtp_modules)})
        self.norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.output = Linear(cfg.dim, cfg.vocab_size)

    def _precompute(self, device=None):
        c = self.config
        inv = None
        if c.max_seq_len > c.original_seq_len:
            inv = yarn_inv_freq(c.qk_rope_head_dim, c.rope_theta, c.rope_factor, c.original_seq_len, c.beta_fast,
                                c.beta_slow)
            inv = inv.to(device) if device is not None else inv
        return precompute_freqs_cis(c.qk_rope_head_dim, c.max_seq_len, c.rope_theta, inv_freq=inv, device=device)

    def init_states(self, *, buffer_device=None, **kw):
        buffer_device = buffer_device or self.freqs_cis.device
        with torch.device(buffer_device):
            self.freqs_cis = self._precompute(buffer_device)
        if self.tok_embeddings is not None:
            self.tok_embeddings.init_states()
        for layer in list(self.layers.values()) + list(self.mtp_layers.values()):
            if layer is not None:
                layer.init_states(buffer_device=buffer_device)
        if self.norm is not None:
            self.norm.init_states()
        if self.output is not None:
            std = self.config.dim ** -0.5
            nn.init.trunc_normal_(self.output.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)

    def forward(self, tokens, attention_masks=None, positions=None):
        n_mtp = len(self.mtp_layers)
        if n_mtp and self.tok_embeddings is not None:
            # the loader hands seq_len + num_mtp tokens; depth k sees tokens shifted by k
            main_tokens = tokens[:, : tokens.shape[1] - n_mtp]
        else:
            main_tokens = tokens
        h = self.tok_embeddings(main_tokens) if self.tok_embeddings is not None else main_tokens
        for layer in self.layers.values():
            h = layer(h, self.freqs_cis, attention_masks, positions)
        if self.norm is None:
            return h
        logits = [self.output(self.norm(h))] if self.output is not None else [self.norm(h)]
        s = main_tokens.shape[1]
        for k, mtp in enumerate(self.mtp_layers.values()):
            emb = self.tok_embeddings(tokens[:, k + 1: k + 1 + s])
            h, hn = mtp(h, emb, self.freqs_cis, attention_masks, positions)
            logits.append(self.output(hn))
        return logits if n_mtp else logits[0]
