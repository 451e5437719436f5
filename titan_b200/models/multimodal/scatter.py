"""Write visual embeddings into the image-placeholder slots of the text embedding sequence.

Parity: torchtitan_npu/models/multimodal/scatter.py:10-74.
"""

from __future__ import annotations

import torch

__all__ = ["scatter_visual_embeddings"]


def scatter_visual_embeddings(hidden_states: torch.Tensor, tokens: torch.Tensor, visual_embeddings: torch.Tensor,
                              visual_token_mask: torch.Tensor, image_token_id: int, *,
                              validate_token_count: bool = True) -> torch.Tensor:
    """hidden_states ``(B, S, D)``, tokens ``(B, S)``, visual_embeddings ``(images, patches, D)``, visual_token_mask
    ``(images, patches)`` bool.  The valid patch embeddings, in order, replace the placeholder positions, in order.
    ``validate_token_count`` compares both counts (one host synchronisation)."""
    if hidden_states.dim() != 3:
        raise ValueError(f"hidden_states must have shape (batch, seq_len, dim), got {tuple(hidden_states.shape)}")
    if tokens.shape != hidden_states.shape[:2]:
        raise ValueError(f"tokens must have shape {tuple(hidden_states.shape[:2])}, got {tuple(tokens.shape)}")
    if visual_embeddings.dim() != 3:
        raise ValueError("visual_embeddings must have shape (num_images, image_seq_len, dim), got "
                         f"{tuple(visual_embeddings.shape)}")
    if visual_token_mask.shape != visual_embeddings.shape[:2]:
        raise ValueError(f"visual_token_mask must have shape {tuple(visual_embeddings.shape[:2])}, got "
                         f"{tuple(visual_token_mask.shape)}")
    if visual_token_mask.dtype != torch.bool:
        raise ValueError(f"visual_token_mask must have dtype torch.bool, got {visual_token_mask.dtype}")
    dim = hidden_states.shape[-1]
    if visual_embeddings.shape[-1] != dim:
        raise ValueError(f"visual_embeddings hidden dim {visual_embeddings.shape[-1]} != hidden_states hidden dim {dim}")
    slots = (tokens == image_token_id).unsqueeze(-1).to(hidden_states.device)
    source = visual_embeddings.to(device=hidden_states.device, dtype=hidden_states.dtype)
    flat = torch.masked_select(source, visual_token_mask.to(hidden_states.device).unsqueeze(-1))
    if validate_token_count:
        n_vis, n_slots = flat.numel() // dim, int(slots.sum().item())
        if n_vis != n_slots:
            raise ValueError(f"Different number of visual embeddings {n_vis} with placeholder in input token "
                             f"embeddings {n_slots}")
    return hidden_states.masked_scatter(slots, flat)
