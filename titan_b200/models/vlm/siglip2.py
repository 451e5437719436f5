"""Siglip2 vision encoder over pre-patchified, zero-padded image batches.

``pixels`` is ``(images, patches, patch_dim)`` (NaFlex layout: every image is a variable-length list of flattened
patches, padded to the longest), ``grid_hw`` is ``(images, patches, 2)`` with the (row, column) of every patch and
`PADDED_PATCH_COORDINATE` on padding.  The learned ``n_pos × n_pos`` position table is resized (bilinear, antialiased) to
each image's grid; padded rows keep a zero position embedding.

Parity: torchtitan_npu/models/vlm/siglip2.py:24-203 on top of the upstream Siglip2 encoder.
"""

from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from titan_b200.models.common.layers import LayerNorm, Linear
from titan_b200.models.multimodal import DenseMaskSDPA
from titan_b200.protocols.module import Module, ModuleDict

__all__ = ["VisionTransformer", "VisionEmbeddings", "resize_positional_embeddings_zero_padded"]


def resize_positional_embeddings_zero_padded(pos_embeddings: torch.Tensor, spatial_shapes: torch.Tensor,
                                             max_length: int) -> torch.Tensor:
    """pos_embeddings ``(h, w, d)``; spatial_shapes ``(images, 2)`` → ``(images, max_length, d)``."""
    out = pos_embeddings.new_zeros((spatial_shapes.shape[0], max_length, pos_embeddings.shape[-1]))
    if spatial_shapes.is_meta:
        # shapes only (memory simulation): the grid sizes are values; the result depends on the table through one
        # interpolation per distinct size, which the differentiable stand-in below represents
        return out + pos_embeddings.reshape(-1, pos_embeddings.shape[-1]).sum(0)
    table = pos_embeddings.permute(2, 0, 1).unsqueeze(0)  # 1 d h w
    by_shape: dict[tuple[int, int], list[int]] = defaultdict(list)
    for i, (h, w) in enumerate(spatial_shapes.tolist()):
        if h > 0 and w > 0:
            by_shape[(int(h), int(w))].append(i)
    for (h, w), idx in by_shape.items():
        r = F.interpolate(table, size=(h, w), mode="bilinear", align_corners=False, antialias=True)
        out[idx, : h * w] = r[0].permute(1, 2, 0).reshape(h * w, -1)
    return out


class VisionEmbeddings(Module):
    def __init__(self, cfg: "VisionTransformer.Config"):
        super().__init__()
        self.n_pos_embs = cfg.n_pos_embs
        self.patch_embedding = Linear(cfg.n_channels * cfg.patch_size * cfg.patch_size, cfg.dim, bias=True)
        self.position_embedding = nn.Embedding(cfg.n_pos_embs ** 2, cfg.dim)

    def forward(self, pixels: torch.Tensor, grid_hw: torch.Tensor) -> torch.Tensor:
        patches = self.patch_embedding(pixels)
        table = self.position_embedding.weight.reshape(self.n_pos_embs, self.n_pos_embs, -1)
        shapes = torch.stack([grid_hw[:, :, 0].amax(dim=1) + 1, grid_hw[:, :, 1].amax(dim=1) + 1], dim=-1).long()
        return patches + resize_positional_embeddings_zero_padded(table, shapes, pixels.shape[1]).to(patches.dtype)

    def init_states(self, **kw):
        self.patch_embedding.init_states()
        nn.init.normal_(self.position_embedding.weight, std=0.02)


class VisionAttention(Module):
    def __init__(self, cfg: "VisionTransformer.Config"):
        super().__init__()
        self.head_dim = cfg.dim // cfg.n_heads
        self.q_proj = Linear(cfg.dim, cfg.dim, bias=True)
        self.k_proj = Linear(cfg.dim, cfg.dim, bias=True)
        self.v_proj = Linear(cfg.dim, cfg.dim, bias=True)
        self.out_proj = Linear(cfg.dim, cfg.dim, bias=True)
        self.inner_attention = DenseMaskSDPA()

    def forward(self, x, attention_masks):
        b, s, _ = x.shape
        q = self.q_proj(x).view(b, s, -1, self.head_dim).transpose(1, 2)
        k = self.k_proj(x).view(b, s, -1, self.head_dim).transpose(1, 2)
        v = self.v_proj(x).view(b, s, -1, self.head_dim).transpose(1, 2)
        o = self.inner_attention(q, k, v, attn_mask=attention_masks)
        return self.out_proj(o.transpose(1, 2).reshape(b, s, -1))

    def init_states(self, **kw):
        for lin in (self.q_proj, self.k_proj, self.v_proj, self.out_proj):
            lin.init_states()


class VisionMLP(Module):
    def __init__(self, cfg: "VisionTransformer.Config"):
        super().__init__()
        self.fc1 = Linear(cfg.dim, cfg.ffn_dim, bias=True)
        self.fc2 = Linear(cfg.ffn_dim, cfg.dim, bias=True)

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(x), approximate="tanh"))

    def init_states(self, **kw):
        self.fc1.init_states()
        self.fc2.init_states()


class VisionLayer(Module):
    def __init__(self, cfg: "VisionTransformer.Config"):
        super().__init__()
        self.layer_norm1 = LayerNorm(cfg.dim, eps=cfg.layer_norm_eps)
        self.self_attn = VisionAttention(cfg)
        self.layer_norm2 = LayerNorm(cfg.dim, eps=cfg.layer_norm_eps)
        self.mlp = VisionMLP(cfg)

    def forward(self, x, attention_masks):
        x = x + self.self_attn(self.layer_norm1(x), attention_masks)
        return x + self.mlp(self.layer_norm2(x))

    def init_states(self, **kw):
        for m in (self.layer_norm1, self.self_attn, self.layer_norm2, self.mlp):
            m.init_states()


class VisionTransformer(Module):
    @dataclass(kw_only=True)
    class Config(Module.Config):
        dim: int = 768
        ffn_dim: int = 3072
        n_layers: int = 12
        n_heads: int = 12
        n_pos_embs: int = 16
        n_channels: int = 3
        patch_size: int = 16
        layer_norm_eps: float = 1e-6
        attn_mask_type: str = "causal"  # causal | full (over valid patches)

    def __init__(self, cfg: "VisionTransformer.Config"):
        super().__init__()
        self.config = cfg
        self.attn_mask_type = cfg.attn_mask_type
        self.embeddings = VisionEmbeddings(cfg)
        self.layers = ModuleDict({str(i): VisionLayer(cfg) for i in range(cfg.n_layers)})
        self.post_layernorm = LayerNorm(cfg.dim, eps=cfg.layer_norm_eps)

    def forward(self, pixel_values, pixel_masks, grid_hw, attention_masks):
        h = self.embeddings(pixel_values, grid_hw)
        for layer in self.layers.values():
            h = layer(h, attention_masks)
        return self.post_layernorm(h)

    def init_states(self, **kw):
        self.embeddings.init_states()
        for layer in self.layers.values():
            layer.init_states()
        self.post_layernorm.init_states()
