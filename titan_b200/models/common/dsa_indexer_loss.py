"""DeepSeek sparse-attention (DSA) indexer loss: KL(teacher ‖ indexer) over the selected keys.

* teacher  = main-attention probability mass summed over heads, gathered at the top-k selected keys and
  renormalised over them (detached from the main graph);
* student  = softmax of the lightning-indexer scores over the same selected keys;
* loss     = mean over queries of ``target_sum · Σ_k t_k (log t_k − log s_k)``; rows without teacher mass
  contribute nothing and keep logits finite.

`DSAIndexerLossAutoScaler` attaches the auxiliary loss to the main graph without changing the forward value:
its backward feeds a constant ``LOSS_SCALE`` into the loss, so the indexer trains from the KL term while the
main loss trains everything else.  `DSAIndexerLossLoggingHelper` accumulates per-layer values for the log line.

Parity: torchtitan_npu/models/common/dsa_indexer_loss.py:22-160.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from titan_b200.protocols.module import Module
from titan_b200.utils.logging import logger

__all__ = ["DSAIndexerLoss", "DSAIndexerLossAutoScaler", "DSAIndexerLossLoggingHelper", "dsa_indexer_loss"]


def dsa_indexer_loss(selected_main_attn_dist: torch.Tensor, index_score: torch.Tensor, loss_scale: float = 1.0,
                     eps: float = 1e-8) -> torch.Tensor:
    t = selected_main_attn_dist.float().clamp_min(0)
    target_sum = t.sum(dim=-1, keepdim=True)
    valid = target_sum > eps
    score = torch.where(valid, index_score, torch.zeros_like(index_score))
    logp = F.log_softmax(score, dim=-1, dtype=torch.float32)
    t = t / target_sum.clamp_min(eps)
    pos = t > 0
    logp = torch.where(pos, logp, torch.zeros_like(logp))
    loss = (t * (t.clamp_min(eps).log() - logp)).sum(dim=-1)
    return (target_sum.squeeze(-1) * loss).mean() * loss_scale


class DSAIndexerLoss(Module):
    def __init__(self, eps: float = 1e-8):
        super().__init__()
        self.eps = eps

    def forward(self, selected_main_attn_dist, index_score, topk_indices=None, loss_scale: float = 1.0):
        return dsa_indexer_loss(selected_main_attn_dist, index_score, loss_scale, self.eps)


class DSAIndexerLossAutoScaler(torch.autograd.Function):
    """Identity on `output`; backward sends ``LOSS_SCALE`` into `loss` (the auxiliary loss rides along)."""

    LOSS_SCALE: torch.Tensor | float = 1.0

    @staticmethod
    def forward(ctx, output: torch.Tensor, loss: torch.Tensor):
        ctx.save_for_backward(loss)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (loss,) = ctx.saved_tensors
        scale = DSAIndexerLossAutoScaler.LOSS_SCALE
        g = torch.ones_like(loss) * (scale if not torch.is_tensor(scale) else scale.to(loss.device))
        return grad_output, g

    @staticmethod
    def set_loss_scale(scale) -> None:
        """``1 / (grad-accumulation steps · size of the loss mesh)``, set once by the trainer."""
        DSAIndexerLossAutoScaler.LOSS_SCALE = scale


class DSAIndexerLossLoggingHelper:
    tracker: dict = {}

    @staticmethod
    def save_loss_to_tracker(loss: torch.Tensor, layer_id: int, num_layers: int) -> None:
        if layer_id is None:
            return
        t = DSAIndexerLossLoggingHelper.tracker
        if "values" not in t or t["values"].numel() != num_layers or t["values"].device != loss.device:
            t["values"] = torch.zeros(num_layers, device=loss.device)
        t["values"][layer_id] += loss.detach().float().reshape(())

    @staticmethod
    def clean_loss_in_tracker() -> None:
        v = DSAIndexerLossLoggingHelper.tracker.get("values")
        if v is not None:
            v.zero_()

    @staticmethod
    def reduce_and_pop(total_acc_steps: int, loss_mesh=None, pp_mesh=None) -> float | None:
        """Mean over layers that produced a loss, after ONE all-reduce of the per-layer vector (log steps only)."""
        v = DSAIndexerLossLoggingHelper.tracker.get("values")
        if v is None:
            return None
        vals = v.clone()
        if loss_mesh is not None:
            import torch.distributed as dist

            dist.all_reduce(vals, op=dist.ReduceOp.AVG if vals.is_cuda else dist.ReduceOp.SUM,
                            group=loss_mesh.get_group())
            if not vals.is_cuda:
                vals /= loss_mesh.size()
        if pp_mesh is not None:
            import torch.distributed as dist

            dist.all_reduce(vals, op=dist.ReduceOp.SUM, group=pp_mesh.get_group())
        valid = vals != 0
        DSAIndexerLossLoggingHelper.clean_loss_in_tracker()
        if int(valid.sum()) == 0:
            return None
        out = float((vals[valid] / max(total_acc_steps, 1)).mean())
        logger.info("indexer loss: %.6f", out)
        return out
