"""Building blocks shared by multimodal models: dense masks, visual-embedding scatter, dense-mask attention core."""

from titan_b200.models.multimodal.attention import DenseMaskSDPA
from titan_b200.models.multimodal.masks import (
    PADDED_PATCH_COORDINATE,
    build_causal_mask,
    build_document_ids,
    build_encoder_causal_mask,
    build_encoder_full_mask,
    build_text_document_causal_mask,
    build_valid_patch_mask,
)
from titan_b200.models.multimodal.scatter import scatter_visual_embeddings

__all__ = ["DenseMaskSDPA", "PADDED_PATCH_COORDINATE", "build_causal_mask", "build_document_ids",
           "build_encoder_causal_mask", "build_encoder_full_mask", "build_text_document_causal_mask",
           "build_valid_patch_mask", "scatter_visual_embeddings"]
