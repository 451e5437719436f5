"""Qwen3 decoder: GQA attention with per-head q/k RMSNorm, half-rotate RoPE, SwiGLU FFN or token-choice MoE,
optional tied embeddings.

Parameter names match the layout the reference's recipes train (``layers.N.attention.{wq,wk,wv,wo,q_norm,k_norm}``,
``layers.N.feed_forward.*`` or ``layers.N.moe.*``), so DCP checkpoints and the Hugging Face adapter line up.

``inner_attention`` is the swap point: the default is the library SDPA core (causal, or a block-causal mask built from
document boundaries); `VarlenAttention` (packed "TND" layout) replaces it in the variable-length recipes, and context
parallelism (Ulysses) hooks it.

Parity: the upstream Qwen3 model the reference re-exports (torchtitan_npu/models/qwen3/__init__.py:15-28) with its
NPU varlen attention (models/common/npu_varlen_attention.py) and recipes (models/qwen3/config_registry.py).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn

from titan_b200.models.common.layers import Embedding, FeedForward, Linear, RMSNorm, ScaledDotProductAttention
from titan_b200.models.common.moe import MoE, MoEArgs
from titan_b200.models.common.rope import apply_rotary_emb_cos_sin, precompute_rope_cache
from titan_b200.protocols.module import BaseModelConfig, Module, ModuleDict

__all__ = ["Qwen3Model", "Qwen3Attention", "Qwen3Block", "block_causal_mask"]


def block_causal_mask(positions: torch.Tensor) -> torch.Tensor:
    """Boolean ``[B, 1, S, S]`` mask for packed documents: position ids restart at 0 at each document start; a query
    sees earlier tokens of its own document only."""
    if positions.dim() == 1:
        positions = positions.unsqueeze(0)
    starts = (positions == 0).cumsum(dim=-1)  # document id per token
    same = starts.unsqueeze(-1) == starts.unsqueeze(-2)
    s = positions.shape[-1]
    causal = torch.ones(s, s, dtype=torch.bool, device=positions.device).tril()
    return (same & causal).unsqueeze(1)


class Qwen3Attention(Module):
    def __init__(self, cfg: "Qwen3Model.Config"):
        super().__init__()
        self.n_heads, self.n_kv_heads, self.head_dim = cfg.n_heads, cfg.n_kv_heads or cfg.n_heads, cfg.head_dim
        self.mask_type = cfg.mask_type
        self.wq = Linear(cfg.dim, self.n_heads * self.head_dim, bias=False)
        self.wk = Linear(cfg.dim, self.n_kv_heads * self.head_dim, bias=False)
        self.wv = Linear(cfg.dim, self.n_kv_heads * self.head_dim, bias=False)
        self.wo = Linear(self.n_heads * self.head_dim, cfg.dim, bias=False)
        self.q_norm = RMSNorm(self.head_dim, eps=cfg.norm_eps) if cfg.qk_norm else None
        self.k_norm = RMSNorm(self.head_dim, eps=cfg.norm_eps) if cfg.qk_norm else None
        if cfg.mask_type == "varlen":
            from titan_b200.models.common.varlen_attention import VarlenAttention

            self.inner_attention = VarlenAttention()
        else:
            self.inner_attention = ScaledDotProductAttention(causal=True)

    def init_states(self, *, init_std: float = 0.02, **kw):
        for lin in (self.wq, self.wk, self.wv):
            lin.init_states(init_std=0.02)
        self.wo.init_states(init_std=init_std)
        for n in (self.q_norm, self.k_norm):
            if n is not None:
                n.init_states()

    def forward(self, x, rope_cache, attention_masks=None, positions=None):
        bs, seqlen, _ = x.shape
        xq = self.wq(x).view(bs, seqlen, -1, self.head_dim)
        xk = self.wk(x).view(bs, seqlen, -1, self.head_dim)
        xv = self.wv(x).view(bs, seqlen, -1, self.head_dim)
        if self.q_norm is not None:
            xq, xk = self.q_norm(xq), self.k_norm(xk)
        xq, xk = apply_rotary_emb_cos_sin(xq, xk, rope_cache, positions)
        out = self.inner_attention(xq.transpose(1, 2), xk.transpose(1, 2), xv.transpose(1, 2),
                                   attn_mask=attention_masks)
        return self.wo(out.transpose(1, 2).contiguous().view(bs, seqlen, -1))


class Qwen3Block(Module):
    def __init__(self, layer_id: int, cfg: "Qwen3Model.Config"):
        super().__init__()
        self.layer_id = layer_id
        self.attention = Qwen3Attention(cfg)
        self.moe_enabled = cfg.moe_enabled
        if self.moe_enabled:
            self.moe = MoE(cfg.dim, cfg.moe_inter_dim, cfg.moe_args)
        else:
            self.feed_forward = FeedForward(dim=cfg.dim, hidden_dim=cfg.hidden_dim)
        self.attention_norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.ffn_norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.weight_init_std = (0.02 / (2 * (layer_id + 1)) ** 0.5) if cfg.depth_init else \
            (0.02 / (2 * cfg.n_layers) ** 0.5)

    def forward(self, x, rope_cache, attention_masks=None, positions=None):
        h = x + self.attention(self.attention_norm(x), rope_cache, attention_masks, positions)
        ff = self.moe if self.moe_enabled else self.feed_forward
        return h + ff(self.ffn_norm(h))

    def init_states(self, *, buffer_device=None, **kw):
        self.attention_norm.init_states()
        self.ffn_norm.init_states()
        self.attention.init_states(init_std=self.weight_init_std)
        if self.moe_enabled:
            self.moe.init_states(init_std=self.weight_init_std, buffer_device=buffer_device)
        else:
            self.feed_forward.init_states(init_std=self.weight_init_std)


class Qwen3Model(Module):
    @dataclass(kw_only=True)
    class Config(BaseModelConfig):
        dim: int = 1024
        n_layers: int = 28
        n_heads: int = 16
        n_kv_heads: int | None = 8
        head_dim: int = 128
        hidden_dim: int = 3072
        vocab_size: int = 151936
        norm_eps: float = 1e-6
        rope_theta: float = 1_000_000.0
        qk_norm: bool = True
        max_seq_len: int = 4096
        depth_init: bool = True
        enable_weight_tying: bool = False
        mask_type: str = "causal"  # causal | block_causal (packed documents; needs `positions`)
        moe_enabled: bool = False
        moe_inter_dim: int = 768
        moe_args: MoEArgs = field(default_factory=lambda: MoEArgs(
            num_experts=128, num_shared_experts=0, top_k=8, score_func="softmax", route_norm=True, route_scale=1.0,
            score_before_experts=False))

        def update_from_config(self, *, trainer_config, **kw) -> None:
            self.max_seq_len = trainer_config.training.seq_len
            self.moe_args._debug_force_load_balance = trainer_config.debug.moe_force_load_balance
            if self.enable_weight_tying and trainer_config.parallelism.pipeline_parallel_degree > 1:
                raise NotImplementedError("tied embeddings cannot be split over pipeline stages")

        def get_nparams_and_flops(self, model, seq_len):
            nparams = emb = routed = 0
            for name, p in model.named_parameters():
                nparams += p.numel()
                if "tok_embeddings" in name:
                    emb += p.numel()
                elif ".moe.experts." in name:
                    routed += p.numel()
            active = nparams - emb - routed
            if routed:
                active += routed * self.moe_args.top_k // self.moe_args.num_experts
            if self.enable_weight_tying:
                active += emb  # the tied matrix still does the output projection
            return nparams, 6 * active + 12 * self.n_layers * self.n_heads * self.head_dim * seq_len

    def __init__(self, cfg: "Qwen3Model.Config"):
        super().__init__()
        self.config = cfg
        self.n_layers = cfg.n_layers
        self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim)
        self.register_buffer("rope_cache", self._precompute(), persistent=False)
        self.layers = ModuleDict({str(i): Qwen3Block(i, cfg) for i in range(cfg.n_layers)})
        self.norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.output = Linear(cfg.dim, cfg.vocab_size, bias=False)
        if cfg.enable_weight_tying:
            self.output.weight = self.tok_embeddings.weight

    def _precompute(self, device=None):
        c = self.config
        return precompute_rope_cache(c.head_dim, c.max_seq_len, c.rope_theta, device=device)

    def init_states(self, *, buffer_device=None, **kw):
        buffer_device = buffer_device or self.rope_cache.device
        with torch.device(buffer_device):
            self.rope_cache = self._precompute(buffer_device)
        if self.tok_embeddings is not None:
            self.tok_embeddings.init_states()
        for layer in self.layers.values():
            if layer is not None:
                layer.init_states(buffer_device=buffer_device)
        if self.norm is not None:
            self.norm.init_states()
        if self.output is not None and not self.config.enable_weight_tying:
            std = self.config.dim ** -0.5
            nn.init.trunc_normal_(self.output.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)
        if self.config.enable_weight_tying and self.output is not None and self.tok_embeddings is not None:
            self.output.weight = self.tok_embeddings.weight  # materialisation from meta breaks the tie

    def forward(self, tokens, attention_masks=None, positions=None):
        h = self.tok_embeddings(tokens) if self.tok_embeddings is not None else tokens
        if attention_masks is None and positions is not None:
            if self.config.mask_type == "block_causal":
                attention_masks = block_causal_mask(positions)
            elif self.config.mask_type == "varlen":
                from titan_b200.models.common.varlen_attention import build_varlen_metadata

                attention_masks = build_varlen_metadata(positions)
        for layer in self.layers.values():
            h = layer(h, self.rope_cache, attention_masks, positions)
        h = self.norm(h) if self.norm is not None else h
        return self.output(h) if self.output is not None else h
