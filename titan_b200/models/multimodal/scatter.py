"""Write visual embeddings into the image-placeholder slots of the text embedding sequence.

Parity: torchtitan_npu/models/multimodal/scatter.py:10-74 (same contract; out of place, so autograd sees it).
"""

from __future__ import annotations

import torch

__all__ = ["scatter_visual_embeddings"]


def _check_layout(hidden_states, tokens, visual_embeddings, visual_token_mask) -> None:
    """One pass over the shape / dtype contract; the message lists everything that is off."""
    problems = []
    if hidden_states.dim() != 3:
        problems.append(f"hidden_states is {tuple(hidden_states.shape)}, expected (batch, seq, dim)")
    elif tuple(tokens.shape) != tuple(hidden_states.shape[:2]):
        problems.append(f"tokens is {tuple(tokens.shape)}, expected {tuple(hidden_states.shape[:2])}")
    if visual_embeddings.dim() != 3:
        problems.append(f"visual_embeddings is {tuple(visual_embeddings.shape)}, expected (images, patches, dim)")
    else:
        if tuple(visual_token_mask.shape) != tuple(visual_embeddings.shape[:2]):
            problems.append(f"visual_token_mask is {tuple(visual_token_mask.shape)}, expected "
                            f"{tuple(visual_embeddings.shape[:2])}")
        if hidden_states.dim() == 3 and visual_embeddings.shape[-1] != hidden_states.shape[-1]:
            problems.append(f"embedding widths differ: visual {visual_embeddings.shape[-1]}, text "
                            f"{hidden_states.shape[-1]}")
    if visual_token_mask.dtype != torch.bool:
        problems.append(f"visual_token_mask is {visual_token_mask.dtype}, expected bool")
    if problems:
        raise ValueError("scatter_visual_embeddings: " + "; ".join(problems))


def scatter_visual_embeddings(hidden_states: torch.Tensor, tokens: torch.Tensor, visual_embeddings: torch.Tensor,
                              visual_token_mask: torch.Tensor, image_token_id: int, *,
                              validate_token_count: bool = True) -> torch.Tensor:
    """hidden_states ``(B, S, D)``, tokens ``(B, S)``, visual_embeddings ``(images, patches, D)``, visual_token_mask
    ``(images, patches)`` bool.  The valid patch embeddings, in order, replace the placeholder positions, in order.
    ``validate_token_count`` compares both counts (one host synchronisation)."""
    _check_layout(hidden_states, tokens, visual_embeddings, visual_token_mask)
    dev, dim = hidden_states.device, hidden_states.shape[-1]
    slots = (tokens == image_token_id).unsqueeze(-1).to(dev)
    patches = visual_embeddings.to(device=dev, dtype=hidden_states.dtype)
    valid = torch.masked_select(patches, visual_token_mask.to(dev).unsqueeze(-1))
    if validate_token_count:
        have, want = valid.numel() // dim, int(slots.sum().item())
        if have != want:
            raise ValueError(f"{have} valid visual patch embeddings for {want} image placeholder tokens")
    return hidden_states.masked_scatter(slots, valid)
