"""DeepSeek-V3 family: multi-head latent attention (MLA) + fine-grained MoE.

Attention: optional low-rank query (``wq_a → q_norm → wq_b``), compressed KV latent
(``wkv_a → kv_norm → wkv_b``) with a decoupled rotary key shared by all heads, per-head dims
``qk_nope + qk_rope`` for Q/K and ``v_head_dim`` for V, YaRN-aware softmax scale.
Blocks: the first ``n_dense_layers`` use a dense SwiGLU FFN, the rest a `MoE`.

FQNs (``layers.N.attention.{wq|wq_a,q_norm,wq_b,wkv_a,kv_norm,wkv_b,wo}``,
``layers.N.moe.{router.gate,experts.w1/w2/w3,shared_experts.*,expert_bias}``,
``layers.N.feed_forward.*``) keep the checkpoint layout the reference's adapters expect
(torchtitan_npu/models/deepseek_v3/__init__.py:27-192, state_dict_adapter.py:24-385).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn

from titan_b200.models.common.layers import Embedding, FeedForward, Linear, RMSNorm, ScaledDotProductAttention
from titan_b200.models.common.moe import MoE, MoEArgs
from titan_b200.models.common.rope import apply_rotary_emb_single_complex, precompute_freqs_cis, yarn_inv_freq
from titan_b200.protocols.module import BaseModelConfig, Module, ModuleDict

__all__ = ["DeepSeekV3Model", "MLAttention", "DSV3Block"]


class MLAttention(Module):
    def __init__(self, cfg: "DeepSeekV3Model.Config"):
        super().__init__()
        self.dim, self.n_heads = cfg.dim, cfg.n_heads
        self.q_lora_rank, self.kv_lora_rank = cfg.q_lora_rank, cfg.kv_lora_rank
        self.qk_nope, self.qk_rope, self.v_head_dim = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.qk_head_dim = self.qk_nope + self.qk_rope
        if self.q_lora_rank == 0:
            self.wq = Linear(cfg.dim, self.n_heads * self.qk_head_dim)
        else:
            self.wq_a = Linear(cfg.dim, self.q_lora_rank)
            self.q_norm = RMSNorm(self.q_lora_rank, eps=cfg.norm_eps)
            self.wq_b = Linear(self.q_lora_rank, self.n_heads * self.qk_head_dim)
        self.wkv_a = Linear(cfg.dim, self.kv_lora_rank + self.qk_rope)
        self.kv_norm = RMSNorm(self.kv_lora_rank, eps=cfg.norm_eps)
        self.wkv_b = Linear(self.kv_lora_rank, self.n_heads * (self.qk_nope + self.v_head_dim))
        self.wo = Linear(self.n_heads * self.v_head_dim, cfg.dim)
        self.softmax_scale = self.qk_head_dim ** -0.5
        if cfg.max_seq_len > cfg.original_seq_len:
            mscale = 0.1 * cfg.mscale * math.log(cfg.rope_factor) + 1.0
            self.softmax_scale *= mscale * mscale
        self.inner_attention = ScaledDotProductAttention(causal=True)

    def forward(self, x, freqs_cis, attention_masks=None, positions=None):
        bsz, seqlen, _ = x.shape
        q = self.wq(x) if self.q_lora_rank == 0 else self.wq_b(self.q_norm(self.wq_a(x)))
        q = q.view(bsz, seqlen, -1, self.qk_head_dim)  # -1: local heads under TP
        q_nope, q_pe = torch.split(q, [self.qk_nope, self.qk_rope], dim=-1)
        q_pe = apply_rotary_emb_single_complex(q_pe, freqs_cis, positions)
        q = torch.cat([q_nope, q_pe], dim=-1)

        kv = self.wkv_a(x)
        kv, k_pe = torch.split(kv, [self.kv_lora_rank, self.qk_rope], dim=-1)
        k_pe = apply_rotary_emb_single_complex(k_pe.unsqueeze(2), freqs_cis, positions)
        kv = self.wkv_b(self.kv_norm(kv)).view(bsz, seqlen, -1, self.qk_nope + self.v_head_dim)
        k_nope, v = torch.split(kv, [self.qk_nope, self.v_head_dim], dim=-1)
        n_local = k_nope.shape[2]
        k = torch.cat([k_nope, k_pe.expand(-1, -1, n_local, -1)], dim=-1)
        out = self.inner_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                   scale=self.softmax_scale, attn_mask=attention_masks)
        out = out.transpose(1, 2).contiguous().view(bsz, seqlen, -1)
        return self.wo(out)

    def init_states(self, *, init_std: float = 0.02, **kw):
        for name in ("wq", "wq_a", "wq_b", "wkv_a", "wkv_b"):
            if hasattr(self, name):
                getattr(self, name).init_states(init_std=0.02)
        self.wo.init_states(init_std=init_std)
        self.kv_norm.init_states()
        if self.q_lora_rank > 0:
            self.q_norm.init_states()


class DSV3Block(Module):
    def __init__(self, layer_id: int, cfg: "DeepSeekV3Model.Config"):
        super().__init__()
        self.layer_id = layer_id
        self.attention = MLAttention(cfg)
        self.attention_norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.ffn_norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.moe_enabled = layer_id >= cfg.n_dense_layers
        if self.moe_enabled:
            self.moe = MoE(cfg.dim, cfg.moe_inter_dim, cfg.moe_args, layer_id=layer_id, vocab_size=cfg.vocab_size)
        else:
            self.feed_forward = FeedForward(dim=cfg.dim, hidden_dim=cfg.inter_dim)
        self.weight_init_std = 0.02 / (2 * (layer_id + 1)) ** 0.5

    def forward(self, x, freqs_cis, attention_masks=None, positions=None):
        x = x + self.attention(self.attention_norm(x), freqs_cis, attention_masks, positions)
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


class DeepSeekV3Model(Module):
    @dataclass(kw_only=True)
    class Config(BaseModelConfig):
        dim: int = 2048
        inter_dim: int = 10944
        moe_inter_dim: int = 1408
        n_layers: int = 27
        n_dense_layers: int = 1
        n_heads: int = 16
        vocab_size: int = 102400
        norm_eps: float = 1e-6
        moe_args: MoEArgs = field(default_factory=MoEArgs)
        q_lora_rank: int = 0
        kv_lora_rank: int = 512
        qk_nope_head_dim: int = 128
        qk_rope_head_dim: int = 64
        v_head_dim: int = 128
        max_seq_len: int = 4096
        original_seq_len: int = 4096
        rope_theta: float = 10000.0
        rope_factor: float = 40
        beta_fast: int = 32
        beta_slow: int = 1
        mscale: float = 1.0
        use_grouped_mm: bool = True

        def update_from_config(self, *, trainer_config, **kw) -> None:
            self.max_seq_len = trainer_config.training.seq_len
            self.moe_args._debug_force_load_balance = trainer_config.debug.moe_force_load_balance
            self.moe_args.use_grouped_mm = self.use_grouped_mm

        def get_nparams_and_flops(self, model: nn.Module, seq_len: int):
            nparams = emb = routed = shared_like = 0
            for name, p in model.named_parameters():
                n = p.numel()
                nparams += n
                if "tok_embeddings" in name:
                    emb += n
                elif ".moe.experts." in name:
                    routed += n
            active = nparams - emb - routed + routed * self.moe_args.top_k // max(self.moe_args.num_experts, 1)
            attn = 12 * self.n_layers * self.n_heads * (self.qk_nope_head_dim + self.qk_rope_head_dim
                                                        + self.v_head_dim) // 2 * seq_len
            return nparams, 6 * active + attn

    def __init__(self, cfg: "DeepSeekV3Model.Config"):
        super().__init__()
        self.config = cfg
        self.n_layers = cfg.n_layers
        self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim)
        self.register_buffer("freqs_cis", self._precompute(), persistent=False)
        self.layers = ModuleDict({str(i): DSV3Block(i, cfg) for i in range(cfg.n_layers)})
        self.norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.output = Linear(cfg.dim, cfg.vocab_size)

    def _precompute(self, device=None):
        c = self.config
        inv = None
        if c.max_seq_len > c.original_seq_len:
            inv = yarn_inv_freq(c.qk_rope_head_dim, c.rope_theta, c.rope_factor, c.original_seq_len, c.beta_fast,
                                c.beta_slow)
            if device is not None:
                inv = inv.to(device)
        return precompute_freqs_cis(c.qk_rope_head_dim, c.max_seq_len, c.rope_theta, inv_freq=inv, device=device)

    def init_states(self, *, buffer_device=None, **kw):
        buffer_device = buffer_device or self.freqs_cis.device
        with torch.device(buffer_device):
            self.freqs_cis = self._precompute(buffer_device)
        if self.tok_embeddings is not None:
            self.tok_embeddings.init_states()
        for layer in self.layers.values():
            if layer is not None:
                layer.init_states(buffer_device=buffer_device)
        if self.norm is not None:
            self.norm.init_states()
        if self.output is not None:
            std = self.config.dim ** -0.5
            nn.init.trunc_normal_(self.output.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)

    def forward(self, tokens, attention_masks=None, positions=None):
        h = self.tok_embeddings(tokens) if self.tok_embeddings is not None else tokens
        for layer in self.layers.values():
            h = layer(h, self.freqs_cis, attention_masks, positions)
        h = self.norm(h) if self.norm is not None else h
        return self.output(h) if self.output is not None else h
