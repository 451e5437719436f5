"""Loss functions: next-token cross entropy (summed; the trainer divides by the global
number of valid tokens) and the multi-token-prediction (MTP) weighted sum.

``main_loss + mtp_loss_weight * Σ_k mtp_loss_k / num_mtp``; logits may be BSND
(``[B, S, V]`` with ``[B, S]`` labels) or compact / TND (``[T, V]``).

Parity: torchtitan_npu/patches/torchtitan/loss.py:47-121.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

__all__ = [
    "IGNORE_INDEX",
    "cross_entropy_loss",
    "compact_cross_entropy_loss",
    "multi_token_cross_entropy_loss",
    "build_cross_entropy_loss",
    "build_mtp_loss",
]

IGNORE_INDEX = -100


def cross_entropy_loss(pred: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Sum of token losses; ``pred`` [B, S, V] (any float dtype), ``labels`` [B, S]."""
    return F.cross_entropy(pred.flatten(0, 1).float(), labels.flatten(0, 1), reduction="sum",
                           ignore_index=IGNORE_INDEX)


def compact_cross_entropy_loss(pred: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Same for packed (TND) logits ``[T, V]`` with labels of any shape holding T entries."""
    return F.cross_entropy(pred.float(), labels.reshape(-1), reduction="sum", ignore_index=IGNORE_INDEX)


def _one(pred, labels):
    return compact_cross_entropy_loss(pred, labels) if pred.dim() == 2 else cross_entropy_loss(pred, labels)


def multi_token_cross_entropy_loss(preds, labels: torch.Tensor, *, num_mtp: int, mtp_loss_weight: float):
    """``preds`` = [main_logits, mtp_1_logits, …]; ``labels`` carries `num_mtp` extra shifted tokens.

    Labels have ``S + num_mtp`` columns: head k (0 = main) is supervised by ``labels[:, k : k + S]``.
    """
    if not isinstance(preds, (list, tuple)):
        return _one(preds, labels)
    if labels.dim() == 3:  # packed stream: one row of labels per head, already aligned ([1 + num_mtp, 1, T])
        parts = list(labels.unbind(0))
    elif labels.dim() == 2:
        s = labels.shape[1] - num_mtp
        parts = [labels[:, k: k + s] for k in range(num_mtp + 1)]
    else:
        s = labels.shape[0] - num_mtp
        parts = [labels[k: k + s] for k in range(num_mtp + 1)]
    main = _one(preds[0], parts[0])
    if num_mtp == 0 or len(preds) == 1:
        return main
    extra = sum(_one(p, parts[k + 1]) for k, p in enumerate(preds[1: num_mtp + 1]))
    return main + mtp_loss_weight * extra / num_mtp


def _fused_requested(trainer_config) -> bool:
    if trainer_config is None:
        return False
    from titan_b200.protocols.converter import has_converter

    return has_converter(trainer_config.model_converters.converters, "b200_cross_entropy")


def fused_cross_entropy_loss(pred: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Sum of token losses through the sm_100a kernel (logits stay in their storage dtype)."""
    from titan_b200.ops.cross_entropy import cross_entropy_sum

    return cross_entropy_sum(pred, labels, IGNORE_INDEX, inplace_backward=True)


def build_cross_entropy_loss(compile_config=None, trainer_config=None):
    if _fused_requested(trainer_config):
        return fused_cross_entropy_loss
    loss_fn = cross_entropy_loss
    if compile_config is not None and compile_config.enable and "loss" in compile_config.components:
        loss_fn = torch.compile(loss_fn, backend=compile_config.backend)
    return loss_fn


def build_mtp_loss(compile_config=None, trainer_config=None):
    num_mtp = trainer_config.training.num_mtp_modules if trainer_config is not None else 0
    weight = trainer_config.training.mtp_loss_weight if trainer_config is not None else 0.3

    def loss_fn(preds, labels):
        return multi_token_cross_entropy_loss(preds, labels, num_mtp=num_mtp, mtp_loss_weight=weight)

    if compile_config is not None and compile_config.enable and "loss" in compile_config.components:
        return torch.compile(loss_fn, backend=compile_config.backend)
    return loss_fn
