// Host entry point of the CTA-pair GEMM (kernel: gemm_pair.cuh) and the dispatcher between it and the
// single-CTA engine.
//
//   tb_gemm_auto   C[M,N] = A · B, picking per shape between 256 x 256 tiles on CTA pairs and 128 x 256 tiles on
//                  single CTAs, and for the pair kernel how the last partial wave is cut along the contraction.
//
// The caller may pass a zero-filled workspace (74 x 256 KB of fp32 partial sums + 4 KB of tickets, see
// `tb_gemm_ws_bytes`); without it tail tiles are computed whole.  The workspace is left zero-filled again, so one
// allocation per stream serves every call on that stream; calls that overlap on the GPU need separate workspaces.
#define TBP_DEFINE_KERNEL
#include "gemm_kernel.cuh"
#include "gemm_pair.cuh"

using namespace tbp;

extern "C" int tb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                            long long ldc, int a_mn, int b_mn, int dtype, int out_fp32, int accumulate, int max_ctas,
                            int* status, cudaStream_t st);

namespace {
constexpr long long TILE_WS_BYTES = (long long)TM * TN * 4;
constexpr int TICKET_BYTES = 4096;

// Relative cost of computing `tiles` tiles on `pairs` pairs with the last `tail` tiles cut in `s` parts, in units of
// one whole tile; a part pays a fixed extra for its atomic epilogue and the read-back of the finisher.
double plan_cost(int tiles, int pairs, int full_waves, int s, double part_overhead) {
  const int tail = tiles - full_waves * pairs;
  if (tail < 0) return 1e30;
  if (tail == 0) return full_waves;
  const int rounds = (tail * s + pairs - 1) / pairs;
  return full_waves + rounds * (1.0 / s + (s > 1 ? part_overhead : 0.0));
}
}  // namespace

// Tuning knobs (process-wide): tile rows walked together, ring depth in use (2..STAGES), L2 promotion of the operand
// tensor maps (CUtensorMapL2promotion: 0 none, 1 = 64 B, 2 = 128 B, 3 = 256 B).  Non-positive values restore defaults.
static int g_group_m = 8, g_stages = STAGES, g_promo = 3;
TB_API int tb_gemm_pair_tune(int group_m, int stages, int promo) {
  g_group_m = group_m > 0 ? group_m : 8;
  g_stages = stages >= 2 && stages <= STAGES ? stages : STAGES;
  g_promo = promo >= 0 && promo <= 3 ? promo : 3;
  return 0;
}
TB_API long long tb_gemm_ws_bytes() { return (long long)(tbg::sm_count() / 2) * TILE_WS_BYTES + TICKET_BYTES; }

// policy: 0 = choose, 1 = single-CTA engine, 2 = CTA pairs.  ws may be null (no tail split).
TB_API int tb_gemm_auto(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                        long long ldc, int a_mn, int b_mn, int dtype, int out_fp32, int accumulate, int policy,
                        void* ws, long long ws_bytes, int max_ctas, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return M == 0 || N == 0 ? 0 : TB_ERR_ARG;
  if (dtype != 1 && dtype != 2) return TB_ERR_ARG;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_fp32 ? 4 : 8))) return TB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(C) & 15) != 0) return TB_ERR_ARG;
  const int tiles = ((M + TM - 1) / TM) * ((N + TN - 1) / TN);
  int pairs = max_pairs();
  if (max_ctas > 0 && pairs > max_ctas / 2) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (policy == 0) {
    // pairs pay off once both SMs of most TPCs have a tile; small problems keep the finer 128 x 256 tiles
    const int single_tiles = ((M + 127) / 128) * ((N + 255) / 256);
    policy = (tiles >= pairs / 2 && single_tiles >= tbg::sm_count() / 2) ? 2 : 1;
  }
  if (policy == 1)
    return tb_gemm_bf16(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, dtype, out_fp32, accumulate, max_ctas, status, st);

  CUtensorMap ta, tb_, tc;
  const CUtensorMapDataType dt = tbg::tm_dtype(dtype);
  if (!a_mn) { if (int rc = tbh::make_tmap_2d(&ta, A, dt, 2, M, K, (uint64_t)lda * 2, HM, BK, 3, g_promo)) return rc; }
  else       { if (int rc = tbh::make_tmap_2d(&ta, A, dt, 2, K, M, (uint64_t)lda * 2, 64, 64, 3, g_promo)) return rc; }
  if (!b_mn) { if (int rc = tbh::make_tmap_2d(&tb_, B, dt, 2, N, K, (uint64_t)ldb * 2, HN, BK, 3, g_promo)) return rc; }
  else       { if (int rc = tbh::make_tmap_2d(&tb_, B, dt, 2, K, N, (uint64_t)ldb * 2, 64, 64, 3, g_promo)) return rc; }
  PairParams p = {};
  p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn; p.out_fp32 = out_fp32; p.is_bf16 = dtype == 1;
  p.accumulate = accumulate; p.ldc = ldc; p.C = C; p.status = status;
  p.group_m = g_group_m; p.stages = g_stages;
  if (!out_fp32 && !accumulate) {
    if (int rc = tbh::make_tmap_2d(&tc, C, dt, 2, M, N, (uint64_t)ldc * 2, HM, 64, 3)) return rc;
    p.tma_store = 1;
  } else {
    tc = ta;  // unused by the kernel
  }
  if (pairs > tiles) pairs = tiles;
  p.full_tiles = tiles; p.split = 1;
  const int kblocks = (K + BK - 1) / BK;
  if (ws != nullptr && tiles > 0) {
    const long long cap_tiles = (ws_bytes - TICKET_BYTES) / TILE_WS_BYTES;
    const int waves = tiles / pairs;
    double best = plan_cost(tiles, pairs, waves, 1, 0.0);
    int best_f = waves, best_s = 1;
    const double overhead = 0.06 * 64.0 / (kblocks < 16 ? 16 : kblocks) + 0.04;  // shorter tiles: dearer parts
    for (int f = waves; f >= 0 && f >= waves - 1; --f) {
      const int tail = tiles - f * pairs;
      if (tail <= 0 || tail > cap_tiles || tail > 2 * pairs) continue;
      for (int s = 2; s <= MAX_SPLIT; ++s) {
        if (kblocks / s < 8) break;  // at least 8 k-blocks per part
        const double c = plan_cost(tiles, pairs, f, s, overhead);
        if (c < best - 0.02) { best = c; best_f = f; best_s = s; }
      }
    }
    if (best_s > 1) {
      p.full_tiles = best_f * pairs; p.split = best_s;
      p.ws = reinterpret_cast<float*>(ws);
      p.tickets = reinterpret_cast<unsigned int*>(reinterpret_cast<uint8_t*>(ws) + cap_tiles * TILE_WS_BYTES);
    }
  }
  return launch_pair(ta, tb_, tc, p, pairs, st);
}
