"""Llama-3 decoder (GQA attention, SwiGLU FFN, RMSNorm, complex RoPE).

Parameter names (``tok_embeddings, layers.N.attention.{wq,wk,wv,wo},
layers.N.feed_forward.{w1,w2,w3}, layers.N.{attention_norm,ffn_norm}, norm,
output``) follow the layout that the reference's users reach with
``MODULE=llama3`` (docs/user-guides/quickstart.md:138-146,
scripts/checkpoint_conversion/convert_to_hf.py:131-132), so DCP checkpoints keep
the same FQNs.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn

from titan_b200.models.common.layers import Embedding, FeedForward, Linear, RMSNorm, ScaledDotProductAttention
from titan_b200.models.common.rope import apply_rotary_emb_complex, precompute_freqs_cis
from titan_b200.protocols.module import BaseModelConfig, Module, ModuleDict

__all__ = ["Llama3Model", "TransformerBlock", "Attention"]


def _ffn_hidden(dim: int, multiple_of: int, ffn_dim_multiplier: float | None) -> int:
    hidden = int(2 * (4 * dim) / 3)
    if ffn_dim_multiplier is not None:
        hidden = int(ffn_dim_multiplier * hidden)
    return multiple_of * ((hidden + multiple_of - 1) // multiple_of)


class Attention(Module):
    def __init__(self, cfg: "Llama3Model.Config"):
        super().__init__()
        self.n_heads = cfg.n_heads
        self.n_kv_heads = cfg.n_kv_heads or cfg.n_heads
        self.head_dim = cfg.dim // cfg.n_heads
        self.wq = Linear(cfg.dim, self.n_heads * self.head_dim, bias=False)
        self.wk = Linear(cfg.dim, self.n_kv_heads * self.head_dim, bias=False)
        self.wv = Linear(cfg.dim, self.n_kv_heads * self.head_dim, bias=False)
        self.wo = Linear(self.n_heads * self.head_dim, cfg.dim, bias=False)
        self.inner_attention = ScaledDotProductAttention(causal=True)

    def init_states(self, *, init_std: float = 0.02, **kwargs):
        for lin in (self.wq, self.wk, self.wv):
            lin.init_states(init_std=0.02)
        self.wo.init_states(init_std=init_std)

    def forward(self, x: torch.Tensor, freqs_cis: torch.Tensor, attention_masks=None, positions=None):
        bs, seqlen, _ = x.shape
        xq, xk, xv = self.wq(x), self.wk(x), self.wv(x)
        # -1 instead of n_heads: under TP each rank holds a slice of the heads
        xq = xq.view(bs, seqlen, -1, self.head_dim)
        xk = xk.view(bs, seqlen, -1, self.head_dim)
        xv = xv.view(bs, seqlen, -1, self.head_dim)
        xq, xk = apply_rotary_emb_complex(xq, xk, freqs_cis, positions)
        out = self.inner_attention(
            xq.transpose(1, 2), xk.transpose(1, 2), xv.transpose(1, 2), attn_mask=attention_masks
        )
        out = out.transpose(1, 2).contiguous().view(bs, seqlen, -1)
        return self.wo(out)


class TransformerBlock(Module):
    def __init__(self, layer_id: int, cfg: "Llama3Model.Config"):
        super().__init__()
        self.layer_id = layer_id
        self.attention = Attention(cfg)
        self.feed_forward = FeedForward(
            dim=cfg.dim, hidden_dim=cfg.ffn_hidden or _ffn_hidden(cfg.dim, cfg.multiple_of, cfg.ffn_dim_multiplier)
        )
        self.attention_norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.ffn_norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        if cfg.depth_init:
            self.weight_init_std = 0.02 / (2 * (layer_id + 1)) ** 0.5
        else:
            self.weight_init_std = 0.02 / (2 * cfg.n_layers) ** 0.5

    def forward(self, x, freqs_cis, attention_masks=None, positions=None):
        h = x + self.attention(self.attention_norm(x), freqs_cis, attention_masks, positions)
        return h + self.feed_forward(self.ffn_norm(h))

    def init_states(self, **kwargs):
        self.attention_norm.init_states()
        self.ffn_norm.init_states()
        self.attention.init_states(init_std=self.weight_init_std)
        self.feed_forward.init_states(init_std=self.weight_init_std)


class Llama3Model(Module):
    @dataclass(kw_only=True)
    class Config(BaseModelConfig):
        dim: int = 4096
        n_layers: int = 32
        n_heads: int = 32
        n_kv_heads: int | None = None
        vocab_size: int = 128256
        multiple_of: int = 256
        ffn_dim_multiplier: float | None = None
        ffn_hidden: int | None = None
        """Explicit FFN width; None derives it from multiple_of / ffn_dim_multiplier."""
        norm_eps: float = 1e-5
        rope_theta: float = 10000.0
        rope_scaling: dict | None = field(default=None)
        max_seq_len: int = 131072
        depth_init: bool = True

        def update_from_config(self, *, trainer_config, **kwargs) -> None:
            self.max_seq_len = trainer_config.training.seq_len

        def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, int]:
            nparams = sum(p.numel() for p in model.parameters())
            emb = sum(p.numel() for n, p in model.named_parameters() if "tok_embeddings" in n)
            head_dim = self.dim // self.n_heads
            # 6·N for the matmuls (embedding lookup is not a matmul) + causal-free attention term
            flops = 6 * (nparams - emb) + 12 * self.n_layers * self.n_heads * head_dim * seq_len
            return nparams, flops

    def __init__(self, cfg: "Llama3Model.Config"):
        super().__init__()
        self.config = cfg
        self.vocab_size = cfg.vocab_size
        self.n_layers = cfg.n_layers
        self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim)
        self.register_buffer("freqs_cis", self._precompute(), persistent=False)
        self.layers = ModuleDict({str(i): TransformerBlock(i, cfg) for i in range(cfg.n_layers)})
        self.norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.output = Linear(cfg.dim, cfg.vocab_size, bias=False)

    def _precompute(self, device=None) -> torch.Tensor:
        c = self.config
        return precompute_freqs_cis(c.dim // c.n_heads, c.max_seq_len, c.rope_theta, scaling=c.rope_scaling,
                                    device=device)

    def init_states(self, *, buffer_device: torch.device | None = None, **kwargs):
        buffer_device = buffer_device or self.freqs_cis.device
        with torch.device(buffer_device):
            self.freqs_cis = self._precompute(buffer_device)
        if self.tok_embeddings is not None:
            self.tok_embeddings.init_states()
        for layer in self.layers.values():
            if layer is not None:
                layer.init_states()
        if self.norm is not None:
            self.norm.init_states()
        if self.output is not None:
            final_std = self.config.dim ** -0.5
            cutoff = 3
            nn.init.trunc_normal_(self.output.weight, mean=0.0, std=final_std, a=-cutoff * final_std,
                                  b=cutoff * final_std)

    def forward(self, tokens: torch.Tensor, attention_masks=None, positions=None):
        # tokens may already be hidden states when this is a non-first pipeline stage
        h = self.tok_embeddings(tokens) if self.tok_embeddings is not None else tokens
        for layer in self.layers.values():
            h = layer(h, self.freqs_cis, attention_masks, positions)
        h = self.norm(h) if self.norm is not None else h
        return self.output(h) if self.output is not None else h
