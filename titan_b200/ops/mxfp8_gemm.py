"""Block-scaled MXFP8 GEMM (`csrc/lowp/mxfp8_gemm.cu`): ``C = dequant(A_q, S_a) · dequant(B_q, S_b)ᵀ`` computed by
`tcgen05.mma.kind::mxf8f6f4.block_scale` with the e8m0 scales applied inside the tensor core.

`pack_scale_atoms` lays the ``[rows, K/32]`` scale bytes out the way the kernel's `tcgen05.cp` wants them: atoms of
128 rows × 4 K-blocks (512 bytes, byte ``(row % 32)·16 + (row // 32 % 4)·4 + block % 4``), stored ``[row block][K/128]``.

`mxfp8_grouped_gemm` runs the three products of a grouped-experts layer over expert-sorted rows (groups padded to
multiples of 128 rows, cumulative ends on the device) as ONE launch each, with no host synchronisation:
``GROUP_B_ROWS`` (forward: the tile's expert picks its rows of the stacked weight), ``GROUP_B_SLICE`` (input gradient:
the expert picks a contraction slice of the transposed weight) and ``GROUP_K`` (weight gradient: the contraction runs
over the expert's own rows).

Parity: `npu_quant_matmul` with MX scales as used by torchtitan_npu/patches/torchao_npu/mx_linear.py:26-100.
"""

from __future__ import annotations

import ctypes

import torch

from titan_b200.ops import _lib

__all__ = ["pack_scale_atoms", "mxfp8_gemm", "mxfp8_gemm_supported", "mxfp8_gemm_ref", "mxfp8_grouped_gemm",
           "GROUP_B_ROWS", "GROUP_K", "GROUP_B_SLICE"]

GROUP_B_ROWS, GROUP_K, GROUP_B_SLICE = 1, 2, 3

_DECLARED = False


def pack_scale_atoms(scales: torch.Tensor, order: str = "m0,m1,kb") -> torch.Tensor:
    """[R, K/32] uint8 → [ceil(R/128), K/128, 512] uint8.  Rows are padded with 127 (scale 1.0).  ``order`` names the
    byte order inside an atom from slowest to fastest index (kept as a parameter so a test can pin the layout)."""
    R, kb = scales.shape
    if kb % 4:
        raise ValueError("K must be a multiple of 128 (4 scale blocks per stage)")
    pad = (-R) % 128
    if pad:
        scales = torch.cat([scales, scales.new_full((pad, kb), 127)], dim=0)
    rb = scales.shape[0] // 128
    v = scales.view(rb, 4, 32, kb // 4, 4)  # [row block, m1, m0, stage, block in stage]
    names = {"m1": 1, "m0": 2, "kb": 4}
    dims = [names[n] for n in order.split(",")]
    return v.permute(0, 3, *dims).contiguous().view(rb, kb // 4, 512)


def mxfp8_gemm_supported(M: int, N: int, K: int) -> bool:
    return M > 0 and N > 0 and M % 128 == 0 and N % 8 == 0 and K % 128 == 0


def mxfp8_gemm_ref(aq, sa, bq, sb) -> torch.Tensor:
    """fp32 reference: dequantise both operands (1×32 blocks along K) and multiply."""
    a = aq.float() * torch.exp2(sa.float() - 127.0).repeat_interleave(32, dim=1)
    b = bq.float() * torch.exp2(sb.float() - 127.0).repeat_interleave(32, dim=1)
    return a @ b.t()


def mxfp8_gemm(aq: torch.Tensor, sa: torch.Tensor, bq: torch.Tensor, sb: torch.Tensor, *, packed: bool = False,
               order: str = "m0,m1,kb", tile_n: int = 0) -> torch.Tensor:
    """aq [M, K], bq [N, K] float8_e4m3fn (or uint8 bit patterns); sa [M, K/32], sb [N, K/32] uint8 e8m0 (or, with
    ``packed``, already in atom order) → bf16 [M, N].  ``tile_n``: 128 (two accumulators, epilogue overlapped), 256
    (one accumulator, least operand traffic) or 0 for the library's choice."""
    global _DECLARED
    M, K = aq.shape
    N = bq.shape[0]
    if aq.is_meta and mxfp8_gemm_supported(M, N, K):   # shapes only (memory simulation)
        _lib.note_skipped_launch("tb_mxfp8_gemm", (None, None, None, None, None, M, N, K))
        return torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
    if not (aq.is_cuda and mxfp8_gemm_supported(M, N, K)):
        raise ValueError(f"mxfp8_gemm: unsupported problem M={M} N={N} K={K} on {aq.device}")
    if not _DECLARED:
        P, I = ctypes.c_void_p, ctypes.c_int
        _lib.declare("tb_mxfp8_gemm", [P, P, P, P, P, I, I, I, I, P, P])
        _DECLARED = True
    if not packed:
        sa, sb = pack_scale_atoms(sa, order), pack_scale_atoms(sb, order)
    aq, bq = aq.contiguous(), bq.contiguous()
    out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
    rc = _lib.lib().tb_mxfp8_gemm(aq.data_ptr(), bq.data_ptr(), sa.data_ptr(), sb.data_ptr(), out.data_ptr(), M, N, K,
                                  int(tile_n), _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "mxfp8_gemm")
    return out


def mxfp8_grouped_gemm(aq: torch.Tensor, sa: torch.Tensor, bq: torch.Tensor, sb: torch.Tensor, offs: torch.Tensor,
                       mode: int, *, tile_n: int = 0, out: torch.Tensor | None = None,
                       packed: bool = False) -> torch.Tensor:
    """Grouped block-scaled GEMM; ``offs`` int32 [E] on the device, cumulative group ends, every group a multiple of
    128 rows.  Operands are quantised along their last dim, scales ``[rows, last/32]`` uint8 (packed here) or, with
    ``packed``, already in atom order (`mx_quantize_dual(..., atoms=True)`).

    * ``GROUP_B_ROWS``:  aq [T, K], bq [E*N, K]  → [T, N]     (N % 128 == 0)
    * ``GROUP_B_SLICE``: aq [T, K], bq [N, E*K]  → [T, N]
    * ``GROUP_K``:       aq [M, T], bq [N, T]    → [E*M, N]   (contraction over each group's rows)

    Rows of the output past the last group, and the weight gradient of an expert without rows, are zeros.  ``out``
    (bf16, contiguous, at least as many rows as the result) receives the result in its leading rows."""
    global _GROUPED_DECLARED
    E = offs.numel()
    if offs.dtype != torch.int32 or not (offs.is_cuda or offs.is_meta):
        raise ValueError("mxfp8_grouped_gemm: offs must be an int32 tensor on the device")
    M, K = aq.shape
    if mode == GROUP_B_ROWS:
        N, rows_out = bq.shape[0] // E, M
        ok = bq.shape[0] == E * N and bq.shape[1] == K and N % 128 == 0
    elif mode == GROUP_B_SLICE:
        N, rows_out = bq.shape[0], M
        ok = bq.shape[1] == E * K
    elif mode == GROUP_K:
        N, rows_out = bq.shape[0], E * M
        ok = bq.shape[1] == K
    else:
        raise ValueError(f"mxfp8_grouped_gemm: unknown mode {mode}")
    if ok and aq.is_meta and mxfp8_gemm_supported(M, N, K):   # shapes only (memory simulation)
        _lib.note_skipped_launch("tb_mxfp8_grouped_gemm", (None, None, None, None, None, M, N, K))
        return out if out is not None else torch.empty(rows_out, N, dtype=torch.bfloat16, device=aq.device)
    if not (ok and aq.is_cuda and mxfp8_gemm_supported(M, N, K)):
        raise ValueError(f"mxfp8_grouped_gemm: unsupported problem mode={mode} A={tuple(aq.shape)} B={tuple(bq.shape)} E={E}")
    if not _GROUPED_DECLARED:
        P, I = ctypes.c_void_p, ctypes.c_int
        _lib.declare("tb_mxfp8_grouped_gemm", [P, P, P, P, P, I, I, I, P, I, I, I, P, P])
        _GROUPED_DECLARED = True
    if not packed:
        sa, sb = pack_scale_atoms(sa), pack_scale_atoms(sb)
    aq, bq = aq.contiguous(), bq.contiguous()
    if out is None:
        out = torch.empty(rows_out, N, dtype=torch.bfloat16, device=aq.device)
    elif not (out.dtype == torch.bfloat16 and out.is_contiguous() and out.dim() == 2 and out.shape[1] == N
              and out.shape[0] >= rows_out and out.device == aq.device):
        raise ValueError("mxfp8_grouped_gemm: `out` must be a contiguous bf16 [>= rows, N] tensor on the same device")
    rc = _lib.lib().tb_mxfp8_grouped_gemm(aq.data_ptr(), bq.data_ptr(), sa.data_ptr(), sb.data_ptr(), out.data_ptr(),
                                          M, N, K, offs.data_ptr(), E, int(mode), int(tile_n),
                                          _lib.shared_status().ptr, _lib.stream_ptr())
    _lib.check(rc, "mxfp8_grouped_gemm")
    return out


_GROUPED_DECLARED = False
