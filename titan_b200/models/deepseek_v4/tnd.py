"""Packed ("global TND") batches for DeepSeek-V4: every valid token of a ``[B, S]`` batch of packed documents is moved
into ONE token stream ``[1, T]``; attention, window, compressor and indexer then work per document, everything else
(embeddings, hyper-connections, MoE, norms, heads) is token-local and runs on the stream as it is.

The dataloader supplies ``positions`` (index inside the document; a document starts where the position is 0; -1 marks
padding, which must come last).  From them this module derives

* the request layout: start / end / length of every document in the stream, ``cu_seqlens_q``;
* per compression ratio ``r``: where complete blocks start (positions ``k·r .. k·r + r - 1`` of one document, all
  present), how many compressed keys every document owns (``cu_seqlens_cmp_kv``) and how many tail tokens stay
  uncompressed (``cmp_residual_k``);
* multi-token-prediction inputs and labels: depth ``k`` pairs token ``t`` with the token ``k + 1`` places later only if
  that one belongs to the same document at the consecutive position; otherwise the label is ignored.

Parity: torchtitan_npu/models/deepseek_v4/tnd.py:19-295 (`DeepSeekV4SMLAAttentionMasks`, `build_smla_attention_masks`,
`smla_global_tnd_post_dataloading_process`).  Global TND excludes pipeline and context parallelism
(torchtitan_npu/models/deepseek_v4/parallelize.py:257-268).
"""

from __future__ import annotations

from itertools import count
from typing import Any, NamedTuple

import torch

from titan_b200.trainer.loss import IGNORE_INDEX

__all__ = ["V4PackedLayout", "lengths_to_cu_seqlens", "build_packed_layout", "pack_global_tnd",
           "compressed_block_starts"]

_LAYOUT_IDS = count()


class V4PackedLayout(NamedTuple):
    cu_seqlens_q: torch.Tensor                   # int32 [docs + 1]
    cu_seqlens_ori_kv: torch.Tensor              # raw keys: same as the queries
    cu_seqlens_cmp_kv: dict                      # ratio -> int32 [docs + 1]
    cmp_residual_k: dict                         # ratio -> int32 [docs] tokens after the last complete block
    block_starts_by_ratio: dict                  # ratio -> int64 [blocks] stream index of each complete block's start
    max_seqlen_q: int
    max_seqlen_cmp_kv: dict
    batch_size: int                              # number of documents
    seq_len: int                                 # tokens in the stream
    doc_ranges: tuple                            # ((start, end), ...) host integers, for per-document work
    cache_id: int = -1


def lengths_to_cu_seqlens(lengths: torch.Tensor) -> torch.Tensor:
    return torch.cat((lengths.new_zeros((1,)), torch.cumsum(lengths, dim=0, dtype=lengths.dtype)))


def _ratios(model_args: Any) -> tuple:
    rs = (*model_args.compress_ratios, getattr(model_args, "mtp_layer_compress_ratio", 1))
    return tuple(sorted({r for r in rs if r > 1}))


def compressed_block_starts(flat_positions: torch.Tensor, ratio: int) -> torch.Tensor:
    """Stream indices ``t`` with ``pos[t] % ratio == 0`` whose block ``t .. t + ratio - 1`` is complete: still inside
    the stream and ending at position ``pos[t] + ratio - 1`` (which implies the same document)."""
    n = flat_positions.numel()
    t = torch.arange(n, device=flat_positions.device)
    end = t + ratio - 1
    end_pos = flat_positions[end.clamp_max(n - 1)]
    ok = flat_positions.remainder(ratio).eq(0) & (end < n) & end_pos.eq(flat_positions + ratio - 1)
    return torch.nonzero(ok, as_tuple=False).flatten()


def build_packed_layout(flat_positions: torch.Tensor, model_args: Any) -> V4PackedLayout:
    """Layout of a stream whose per-token document positions are ``flat_positions`` [T] (no padding)."""
    if flat_positions.dim() != 1 or flat_positions.numel() == 0:
        raise ValueError("packed DeepSeek-V4 positions must be a non-empty 1-D tensor")
    pos = flat_positions.long()
    n = pos.numel()
    starts = torch.nonzero(pos.eq(0), as_tuple=False).flatten()
    if starts.numel() == 0 or int(starts[0]) != 0:  # a stream that begins inside a document
        starts = torch.cat((starts.new_zeros((1,)), starts))
    ends = torch.cat((starts[1:], starts.new_tensor((n,))))
    lengths = (ends - starts).to(torch.int32)
    block_starts, cmp_lengths = {}, {}
    for r in _ratios(model_args):
        bs = compressed_block_starts(pos, r).contiguous()
        block_starts[r] = bs
        cmp_lengths[r] = (torch.searchsorted(bs, ends) - torch.searchsorted(bs, starts)).to(torch.int32)
    s_host, e_host = starts.tolist(), ends.tolist()
    return V4PackedLayout(
        cu_seqlens_q=lengths_to_cu_seqlens(lengths),
        cu_seqlens_ori_kv=lengths_to_cu_seqlens(lengths),
        cu_seqlens_cmp_kv={r: lengths_to_cu_seqlens(v) for r, v in cmp_lengths.items()},
        cmp_residual_k={r: lengths - r * v for r, v in cmp_lengths.items()},
        block_starts_by_ratio=block_starts,
        max_seqlen_q=int(lengths.max()),
        max_seqlen_cmp_kv={r: int(v.max()) if v.numel() else 0 for r, v in cmp_lengths.items()},
        batch_size=len(s_host),
        seq_len=n,
        doc_ranges=tuple(zip(s_host, e_host)),
        cache_id=next(_LAYOUT_IDS),
    )


def pack_global_tnd(inputs: torch.Tensor, labels: torch.Tensor, positions: torch.Tensor, model_args: Any):
    """``[B, S + num_mtp]`` packed batch → ``(inputs [1, T], labels, extra_kwargs)``.

    ``labels`` comes back as ``[1, T]`` without MTP and ``[1 + num_mtp, 1, T]`` with it (row 0 the main head);
    ``extra_kwargs`` holds ``positions`` [1, T], ``attention_masks`` (the `V4PackedLayout`) and, with MTP,
    ``mtp_inputs`` [num_mtp, 1, T]."""
    num_mtp = int(getattr(model_args, "num_mtp_modules", 0))
    if inputs.dim() != 2 or inputs.shape != labels.shape or positions.dim() != 2:
        raise RuntimeError("global TND expects [B, S] input and labels of one shape and 2-D positions")
    s = inputs.shape[1] - num_mtp
    if s <= 0:
        raise RuntimeError("global TND: no main-sequence tokens left after removing the MTP tail")
    if positions.shape == (inputs.shape[0], s) and num_mtp > 0:
        # loaders describe the main tokens only: what follows a row is unknown, so it pairs with nothing
        positions = torch.cat([positions, positions.new_full((inputs.shape[0], num_mtp), -1)], dim=1)
    if positions.shape != inputs.shape:
        raise RuntimeError(f"global TND: positions {tuple(positions.shape)} do not describe input "
                           f"{tuple(inputs.shape)}")
    main_pos = positions[:, :s]
    valid = main_pos.ge(0)
    flat_valid = valid.reshape(-1)
    if bool(((torch.cumsum((~valid).int(), dim=1) > 0) & valid).any()):
        raise ValueError("global TND: padding (position -1) must follow the valid tokens of every row")
    if not bool(flat_valid.any()):
        raise RuntimeError("global TND: the batch holds no valid token")
    inputs_tnd = inputs[:, :s][valid].unsqueeze(0)
    pos_tnd = main_pos[valid]
    extra: dict = {}
    if num_mtp > 0:
        doc_of = torch.cumsum(positions.eq(0).int(), dim=1)
        lab, inp = [labels[:, :s][valid]], []
        for k in range(1, num_mtp + 1):
            sh_pos, sh_doc = positions[:, k: k + s], doc_of[:, k: k + s]
            ok = valid & sh_pos.ge(0) & sh_doc.eq(doc_of[:, :s]) & sh_pos.eq(main_pos + k)
            inp.append(torch.where(ok, inputs[:, k: k + s], inputs[:, :s])[valid])
            lab.append(labels[:, k: k + s].masked_fill(~ok, IGNORE_INDEX)[valid])
        labels_tnd = torch.stack(lab, 0).unsqueeze(1)
        extra["mtp_inputs"] = torch.stack(inp, 0).unsqueeze(1)
    else:
        labels_tnd = labels[:, :s][valid].unsqueeze(0)
    # rows are concatenated: a row that does not start with position 0 continues nothing, it opens a document
    row_first = torch.zeros_like(valid)
    row_first[:, 0] = True
    flat_pos = pos_tnd.clone()
    opens = row_first[valid] & flat_pos.ne(0)
    if bool(opens.any()):
        raise ValueError("global TND: every row must start a document (position 0 in its first column)")
    extra["positions"] = flat_pos.unsqueeze(0)
    extra["attention_masks"] = build_packed_layout(flat_pos, model_args)
    return inputs_tnd, labels_tnd, extra
