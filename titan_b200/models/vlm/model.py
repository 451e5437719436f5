"""Llama-3 decoder with a Siglip2 vision tower: image patches are encoded, projected to the text width and written
into the image-placeholder slots of the token embeddings.

Both towers use dense boolean masks: text tokens attend causally within their packed document, patches attend over the
valid patches of their image.  The trainer obtains the masks from `get_attention_masks` once per step.

Parity: `Llama3Siglip2TransformerNpu` (torchtitan_npu/models/vlm/model.py:33-111).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from titan_b200.models.common.layers import Linear
from titan_b200.models.llama3.model import Llama3Model
from titan_b200.models.multimodal import (
    DenseMaskSDPA,
    build_encoder_causal_mask,
    build_encoder_full_mask,
    build_text_document_causal_mask,
    build_valid_patch_mask,
    scatter_visual_embeddings,
)
from titan_b200.models.vlm.siglip2 import VisionTransformer
from titan_b200.protocols.module import Module

__all__ = ["Llama3Siglip2Transformer", "SpecialTokens", "Projector"]


@dataclass
class SpecialTokens:
    img_id: int
    boi_id: int
    eoi_id: int
    pad_id: int
    ignore_id: int = -100


class Projector(Module):
    """Two-layer MLP from the vision width to the text width."""

    def __init__(self, in_dim: int, out_dim: int):
        super().__init__()
        self.w1 = Linear(in_dim, in_dim, bias=True)
        self.w2 = Linear(in_dim, out_dim, bias=True)

    def forward(self, x):
        return self.w2(F.gelu(self.w1(x)))

    def init_states(self, **kw):
        self.w1.init_states()
        self.w2.init_states()


def _grid_hw(grid_thw: torch.Tensor) -> torch.Tensor:
    return grid_thw[:, :, 1:]


class Llama3Siglip2Transformer(Llama3Model):
    @dataclass(kw_only=True)
    class Config(Llama3Model.Config):
        encoder: VisionTransformer.Config = field(default_factory=VisionTransformer.Config)
        img_token_id: int = 1998
        boi_token_id: int = 1999
        eoi_token_id: int = 2000
        pad_token_id: int = 2001
        eos_token_id: int = 2

    def __init__(self, cfg: "Llama3Siglip2Transformer.Config"):
        super().__init__(cfg)
        self.encoder = VisionTransformer(cfg.encoder)
        self.projector = Projector(cfg.encoder.dim, cfg.dim)
        for block in self.layers.values():
            block.attention.inner_attention = DenseMaskSDPA()

    @property
    def special_tokens(self) -> SpecialTokens:
        c = self.config
        return SpecialTokens(img_id=c.img_token_id, boi_id=c.boi_token_id, eoi_id=c.eoi_token_id, pad_id=c.pad_token_id)

    def init_states(self, *, buffer_device=None, **kw):
        super().init_states(buffer_device=buffer_device)
        if self.encoder is not None:
            self.encoder.init_states()
            self.projector.init_states()

    def get_attention_masks(self, input_batch: torch.Tensor, tokenizer=None, extra_inputs: dict | None = None):
        if extra_inputs is None or "grid_thw" not in extra_inputs:
            raise ValueError("VLM dense masks require extra_inputs['grid_thw']")
        eos_id = getattr(tokenizer, "eos_id", None) if tokenizer is not None else self.config.eos_token_id
        if eos_id is None:
            raise ValueError("VLM dense masks require tokenizer.eos_id")
        valid = build_valid_patch_mask(_grid_hw(extra_inputs["grid_thw"]))
        enc = build_encoder_causal_mask(valid) if self.config.encoder.attn_mask_type == "causal" \
            else build_encoder_full_mask(valid)
        return {"llama3_masks": build_text_document_causal_mask(input_batch, eos_id), "encoder_masks": enc,
                "pixel_masks": valid}

    def forward(self, tokens, pixel_values=None, grid_thw=None, special_tokens: SpecialTokens | None = None,
                attention_masks=None, positions=None):
        h = self.tok_embeddings(tokens) if self.tok_embeddings is not None else tokens
        if attention_masks is None:
            attention_masks = self.get_attention_masks(tokens, None, {"grid_thw": grid_thw})
        if self.encoder is not None and pixel_values is not None:
            pixel_masks = attention_masks.get("pixel_masks")
            if pixel_masks is None:
                raise ValueError("VLM dense masks require attention_masks['pixel_masks']")
            vis = self.encoder(pixel_values, pixel_masks, _grid_hw(grid_thw), attention_masks["encoder_masks"])
            vis = self.projector(vis)
            img_id = (special_tokens or self.special_tokens).img_id
            h = scatter_visual_embeddings(h, tokens, vis, pixel_masks, img_id, validate_token_count=False)
        for layer in self.layers.values():
            h = layer(h, self.freqs_cis, attention_masks["llama3_masks"], positions)
        h = self.norm(h) if self.norm is not None else h
        return self.output(h) if self.output is not None else h
