"""Sequence-parallel linears on the fused kernels (async tensor parallelism).

Between transformer sub-layers the activations are sequence-sharded ``[S/tp, D]`` (batch 1 per rank, rows of one
sequence).  Instead of all-gather → GEMM and GEMM → reduce-scatter as separate NCCL + library calls, the column- and
row-parallel linears run on the kernels that move the operand over NVLink while the tensor cores work:

* `ag_multi_linear(x_shard, [w_a, w_b, ...])` – all-gather→GEMM for the first weight (`tb_ag_gemm`: copier CTAs pull
  every remote shard once, tiles wait on per-chunk flags); the gathered activations that kernel leaves behind feed the
  other projections as plain tcgen05 GEMMs.  Backward: ``dX = reduce_scatter([g_a | g_b | ...] · [w_a; w_b; ...])`` is
  ONE GEMM→reduce-scatter over the concatenated contraction dim, the weight gradients are local GEMMs against the saved
  gathered activations.
* `linear_rs(x, w)` – GEMM→reduce-scatter (`tb_gemm_rs`: the epilogue stores each tile into its owner's staging slot,
  `tb_rs_reduce` sums the slots).  Backward: ``dX = all_gather(g_shard) · w`` is an all-gather→GEMM whose gathered
  gradient also serves the weight gradient.

`enable_for_llama` rewires the attention and FFN forwards of a Llama-style model (weights stay the column / row shards
the tensor-parallel plan made: checkpoints are unchanged).  The fused path needs one sequence per rank (local batch 1);
other batches keep the library path.

Parity: the async-TP switch of the reference (`maybe_enable_async_tp`, torchtitan_npu/patches/torch/
micro_pipeline_tp.py:114-144 fuses all-gather + matmul and matmul + reduce-scatter through symmetric memory).
"""

from __future__ import annotations

import types

import torch
import torch.nn.functional as F

from titan_b200.ops import fused_comm

__all__ = ["ag_multi_linear", "linear_rs", "ag_multi_linear_batched", "linear_rs_batched", "enable_for_llama"]


def _mm(a, b_t):
    """a [M, K] · b_tᵀ, b_t [N, K] (tcgen05 GEMM when the operands qualify)."""
    from titan_b200.ops import gemm as G

    if G.supported(a, b_t) and a.shape[1] % 8 == 0:
        return G.gemm(a.contiguous(), b_t.contiguous())
    return a @ b_t.t()


def _mm_tn(a, b):
    """aᵀ · b with a [R, M], b [R, N] → [M, N] (weight-gradient shape: both operands contraction-major)."""
    from titan_b200.ops import gemm as G

    if G.supported(a, b) and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0:
        return G.gemm(a.contiguous(), b.contiguous(), a_mn=True, b_mn=True)
    return a.t() @ b


class _AGMultiLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, group, *weights):
        y0, xg = fused_comm.all_gather_matmul(x_shard, weights[0], group, return_gathered=True)
        outs = [y0] + [_mm(xg, w) for w in weights[1:]]
        ctx.save_for_backward(xg, *weights)
        ctx.group = group
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        xg, *weights = ctx.saved_tensors
        g = torch.cat([gi.contiguous() for gi in grads], dim=1)          # [M, ΣN]
        w_t = torch.cat(list(weights), dim=0).t().contiguous()            # [K, ΣN]
        dx = fused_comm.matmul_reduce_scatter(g, w_t, ctx.group)          # [M / tp, K]
        dws = [_mm_tn(gi.contiguous(), xg) for gi in grads]               # [N_i, K]
        return (dx, None, *dws)


def ag_multi_linear(x_shard: torch.Tensor, weights: list[torch.Tensor], group) -> list[torch.Tensor]:
    """x_shard [S/tp, K]; weights [N_i, K] (local column shards) → outputs [S, N_i]."""
    return list(_AGMultiLinear.apply(x_shard, group, *weights))


class _LinearRS(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group):
        ctx.save_for_backward(x, w)
        ctx.group = group
        return fused_comm.matmul_reduce_scatter(x, w, group)

    @staticmethod
    def backward(ctx, g_shard):
        x, w = ctx.saved_tensors
        dx, gg = fused_comm.all_gather_matmul(g_shard.contiguous(), w.t().contiguous(), ctx.group,
                                              return_gathered=True)          # [M, K_local], gathered grad [M, N]
        return dx, _mm_tn(gg, x), None


def linear_rs(x: torch.Tensor, w: torch.Tensor, group) -> torch.Tensor:
    """x [S, K_local], w [N, K_local] (local row shard) → reduce-scattered [S/tp, N]."""
    return _LinearRS.apply(x, w, group)


def ag_multi_linear_batched(x: torch.Tensor, weights: list[torch.Tensor], group) -> list[torch.Tensor]:
    """x [B, S/tp, K] → outputs [B, S, N_i].  The fused kernel gathers one sequence's rows in rank order, so a batch
    runs one launch per sequence (a single sequence adds no copy)."""
    if x.shape[0] == 1:
        return [y.unsqueeze(0) for y in ag_multi_linear(x[0], weights, group)]
    per_seq = [ag_multi_linear(x[b], weights, group) for b in range(x.shape[0])]
    return [torch.stack([seq[i] for seq in per_seq]) for i in range(len(weights))]


def linear_rs_batched(x: torch.Tensor, w: torch.Tensor, group) -> torch.Tensor:
    """x [B, S, K_local] → reduce-scattered [B, S/tp, N], one launch per sequence."""
    if x.shape[0] == 1:
        return linear_rs(x[0], w, group).unsqueeze(0)
    return torch.stack([linear_rs(x[b], w, group) for b in range(x.shape[0])])


def _local(p):
    return p.to_local() if hasattr(p, "to_local") else p


def enable_for_llama(model, tp_mesh) -> int:
    """Route attention (wq|wk|wv → SDPA → wo) and FFN (w1|w3 → SwiGLU → w2) of every block through the fused
    kernels.  Returns the number of rewired blocks."""
    from titan_b200.models.common.rope import apply_rotary_emb_complex

    group = tp_mesh.get_group()
    fused_comm.enable_for_group(group)

    def attn_forward(self, x, freqs_cis, attention_masks=None, positions=None):
        xq, xk, xv = ag_multi_linear_batched(
            x, [_local(self.wq.weight), _local(self.wk.weight), _local(self.wv.weight)], group)
        b, s = xq.shape[0], xq.shape[1]
        xq = xq.view(b, s, -1, self.head_dim)
        xk = xk.view(b, s, -1, self.head_dim)
        xv = xv.view(b, s, -1, self.head_dim)
        xq, xk = apply_rotary_emb_complex(xq, xk, freqs_cis, positions)
        out = self.inner_attention(xq.transpose(1, 2), xk.transpose(1, 2), xv.transpose(1, 2),
                                   attn_mask=attention_masks)
        out = out.transpose(1, 2).reshape(b, s, -1)
        return linear_rs_batched(out, _local(self.wo.weight), group)

    def ffn_forward(self, x):
        g, u = ag_multi_linear_batched(x, [_local(self.w1.weight), _local(self.w3.weight)], group)
        return linear_rs_batched(F.silu(g) * u, _local(self.w2.weight), group)

    n = 0
    for block in model.layers.values():
        if block is None:
            continue
        block.attention.forward = types.MethodType(attn_forward, block.attention)
        if hasattr(block, "feed_forward"):
            block.feed_forward.forward = types.MethodType(ffn_forward, block.feed_forward)
        n += 1
    return n
