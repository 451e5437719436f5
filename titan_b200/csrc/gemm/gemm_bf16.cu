// Host entry points of the dense and grouped tcgen05 GEMMs (kernel: gemm_kernel.cuh).
//
//   tb_gemm_bf16         C[M,N] = A · B                                  (linear fwd / dgrad / wgrad)
//   tb_grouped_gemm_m    C[rows,N] = A[rows,K] · B[g]  per row group     (MoE experts fwd / dgrad)
//   tb_grouped_gemm_k    C[g][M,N] = A_gᵀ · B_g        per row group     (MoE experts wgrad)
//
// Grouped layouts use cumulative row offsets `offs[g]` (int32, device memory) whose values are
// multiples of 128: the permutation kernel pads every expert's segment, so a tile never straddles two
// experts and padded rows are zero.  No host-device synchronisation is needed: the kernel derives the
// tile count from `offs` on the device and the caller sizes buffers for the worst case.
//
// Replaces `aten::_grouped_mm` → `npu_grouped_matmul` of the reference (ops/_grouped_mm.py:10-42:
// 2D x 3D forward/dgrad and 2D x 2D split-K wgrad with int32 offsets).
#define TBG_DEFINE_KERNEL
#include "gemm_kernel.cuh"

using namespace tbg;

namespace {
void fill_common(GemmParams& p, int mode, int M, int N, int K, int a_mn, int b_mn, int dtype, int out_fp32,
                 int accumulate, long long ldc, void* C, int* status) {
  p = GemmParams{};
  p.mode = mode; p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn; p.out_fp32 = out_fp32;
  p.is_bf16 = dtype == 1; p.accumulate = accumulate; p.ldc = ldc; p.C = C; p.status = status;
  p.nranks = 1;
}
}  // namespace

// dtype: 1 = bf16, 2 = fp16 (A, B and—unless out_fp32—C).  lda/ldb/ldc in elements.
// Requirements: pointers 16-byte aligned; lda, ldb multiples of 8; ldc multiple of 8 (4 for fp32 out).
TB_API int tb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                        long long ldc, int a_mn, int b_mn, int dtype, int out_fp32, int accumulate, int max_ctas,
                        int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return M == 0 || N == 0 ? 0 : TB_ERR_ARG;
  if (dtype != 1 && dtype != 2) return TB_ERR_ARG;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_fp32 ? 4 : 8))) return TB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(C) & 15) != 0) return TB_ERR_ARG;
  AMaps am;
  CUtensorMap tb_;
  if (int rc = make_a_map(&am.m[0], A, dtype, a_mn, (uint64_t)M, (uint64_t)K, lda)) return rc;
  if (int rc = make_b_map(&tb_, B, dtype, b_mn, (uint64_t)N, (uint64_t)K, ldb)) return rc;
  GemmParams p;
  fill_common(p, PLAIN, M, N, K, a_mn, b_mn, dtype, out_fp32, accumulate, ldc, C, status);
  CMaps cm;
  if (!out_fp32 && !accumulate) {
    if (int rc = make_c_map(&cm.m[0], C, dtype, (uint64_t)M, (uint64_t)N, ldc)) return rc;
    p.tma_store = 1;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  return launch(am, tb_, cm, p, grid, st);
}

// A: [rows_cap, K] K-major.  B: b_mn = 0 → [G, N, K];  b_mn = 1 → [G, K, N].  C: [rows_cap, N].
// offs: [G] cumulative padded row ends (multiples of 128, last <= rows_cap).
TB_API int tb_grouped_gemm_m(const void* A, const void* B, void* C, const int* offs, int G, int rows_cap, int N,
                             int K, int b_mn, int dtype, int* status, cudaStream_t st) {
  if (G < 1 || G > MAX_GROUPS || rows_cap <= 0 || N <= 0 || K <= 0) return rows_cap == 0 ? 0 : TB_ERR_ARG;
  if (dtype != 1 && dtype != 2) return TB_ERR_ARG;
  if ((K % 8) || (N % 8)) return TB_ERR_ARG;
  if (b_mn && (K % BK)) return TB_ERR_ARG;  // K rows of consecutive groups are adjacent in the 2-D view of B
  AMaps am;
  CUtensorMap tb_;
  if (int rc = make_a_map(&am.m[0], A, dtype, 0, (uint64_t)rows_cap, (uint64_t)K, K)) return rc;
  if (!b_mn) {
    if (int rc = make_b_map(&tb_, B, dtype, 0, (uint64_t)G * N, (uint64_t)K, K)) return rc;
  } else {
    if (int rc = make_b_map(&tb_, B, dtype, 1, (uint64_t)N, (uint64_t)G * K, N)) return rc;
  }
  GemmParams p;
  fill_common(p, GROUPED_M, rows_cap, N, K, 0, b_mn, dtype, 0, 0, N, C, status);
  p.num_groups = G; p.offs = offs; p.b_group_rows = b_mn ? K : N;
  CMaps cm;
  if (int rc = make_c_map(&cm.m[0], C, dtype, (uint64_t)rows_cap, (uint64_t)N, N)) return rc;
  p.tma_store = 1;  // segments are 128-row aligned: whole tiles always belong to one expert
  return launch(am, tb_, cm, p, sm_count(), st);
}

// dW[g] [M, N] = A[rows of g, M]ᵀ · B[rows of g, N]   (A: [rows_cap, M], B: [rows_cap, N], both row-major)
// C: [G, M, N] in the input dtype (or fp32 when out_fp32).  Groups without rows produce zeros.
TB_API int tb_grouped_gemm_k(const void* A, const void* B, void* C, const int* offs, int G, int rows_cap, int M, int N,
                             int dtype, int out_fp32, int* status, cudaStream_t st) {
  if (G < 1 || G > MAX_GROUPS || M <= 0 || N <= 0 || rows_cap <= 0) return TB_ERR_ARG;
  if (dtype != 1 && dtype != 2) return TB_ERR_ARG;
  if ((M % 8) || (N % 8)) return TB_ERR_ARG;
  AMaps am;
  CUtensorMap tb_;
  if (int rc = make_a_map(&am.m[0], A, dtype, 1, (uint64_t)M, (uint64_t)rows_cap, M)) return rc;
  if (int rc = make_b_map(&tb_, B, dtype, 1, (uint64_t)N, (uint64_t)rows_cap, N)) return rc;
  GemmParams p;
  fill_common(p, GROUPED_K, M, N, rows_cap, 1, 1, dtype, out_fp32, 0, N, C, status);
  p.num_groups = G; p.offs = offs; p.c_group_stride = (long long)M * N;
  CMaps cm;
  if (!out_fp32 && M % BM == 0) {  // otherwise a tile's tail rows would land in the next group's matrix
    if (int rc = make_c_map(&cm.m[0], C, dtype, (uint64_t)G * M, (uint64_t)N, N)) return rc;
    p.tma_store = 1;
  }
  const int tiles = G * ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  return launch(am, tb_, cm, p, tiles < sm_count() ? tiles : sm_count(), st);
}

// Lightning-indexer scores.  q: [S*H, D] (row = query*H + head; H a power of two), k: [T, D], w: [S*H] fp32 weights,
// scores: [S, ld] fp32 with scores[s, t] = Σ_h w[s,h]·relu(q[s,h]·k[t]) for every visible key
// t < (pos_offset + s + 1) / ratio (ratio 1: causal tokens; ratio r: compressed keys, one per r tokens, visible once
// their block is complete).  Entries in the causal future of a query are left unwritten where a whole tile is
// skipped: consumers must not read them.
TB_API int tb_indexer_scores(const void* q, const void* k, const float* w, float* scores, int S, int H, int T, int D,
                             long long ld, int pos_offset, int ratio, int dtype, int* status, cudaStream_t st) {
  if (S <= 0 || T <= 0) return 0;
  if (ratio < 1) return TB_ERR_ARG;
  if (H < 1 || H > BN || (H & (H - 1)) != 0 || D % 8 || (dtype != 1 && dtype != 2)) return TB_ERR_ARG;
  AMaps am;
  CUtensorMap tb_;
  CMaps cm;
  const int N = S * H;  // columns: (query, head) pairs; rows: keys
  if (int rc = make_a_map(&am.m[0], k, dtype, 0, (uint64_t)T, (uint64_t)D, D)) return rc;
  if (int rc = make_b_map(&tb_, q, dtype, 0, (uint64_t)N, (uint64_t)D, D)) return rc;
  GemmParams p;
  fill_common(p, INDEXER, T, N, D, 0, 0, dtype, 0, 0, N, nullptr, status);
  p.idx_weights = w; p.idx_heads = H; p.idx_scores = scores; p.idx_ld = ld; p.idx_pos_offset = pos_offset;
  p.idx_ratio = ratio;
  const int tiles = ((T + BM - 1) / BM) * ((N + BN - 1) / BN);
  return launch(am, tb_, cm, p, tiles < sm_count() ? tiles : sm_count(), st);
}
