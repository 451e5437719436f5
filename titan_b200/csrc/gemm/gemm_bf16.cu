// Persistent, warp-specialised bf16/fp16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   C[M, N] = A · B      A: M x K,  B: K x N   (fp32 accumulation in tensor memory)
//
// Operand storage is chosen per call so that forward, input-gradient and weight-gradient products
// of a linear layer all run without a transpose copy:
//   a_mn = 0 : A stored [M, K] row-major (K-major)      a_mn = 1 : A stored [K, M] row-major (MN-major)
//   b_mn = 0 : B stored [N, K] row-major (K-major)      b_mn = 1 : B stored [K, N] row-major (MN-major)
//   forward  y  = x · Wᵀ   : a_mn 0 (x),  b_mn 0 (W [N,K])
//   dgrad    dx = dy · W   : a_mn 0 (dy), b_mn 1 (W [N,K] is "[K', N']" of this product)
//   wgrad    dW = dyᵀ · x  : a_mn 1 (dy), b_mn 1 (x)
//
// Structure (one CTA per SM, 192 threads):
//   warp 0      TMA producer: global → 128B-swizzled shared tiles, 4-stage ring, mbarrier full/empty
//   warp 1      MMA issuer : one thread issues tcgen05.mma (128 x 256 x 16), accumulators in TMEM,
//               two 256-column accumulator buffers so the epilogue of tile i overlaps the main loop of i+1
//   warps 2..5  epilogue   : tcgen05.ld (32 lanes x 32 columns per warp and step) → convert → global
// Tiles are visited in a grouped order so concurrently running CTAs share operand tiles in L2.
// No multicast is used.  Every wait is time-bounded; on expiry the kernel records a status code,
// raises a CTA-wide abort flag, drains and frees its tensor memory.
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 /*align*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 16;
constexpr int NUM_THREADS = 192;

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;
  int out_fp32;      // 0: C has the input dtype (bf16/fp16), 1: fp32
  int is_bf16;       // input dtype: 1 bf16, 0 fp16
  int accumulate;    // 1: C += A·B (read-modify-write in the epilogue)
  long long ldc;     // elements between rows of C
  void* C;
  int* status;
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// time-bounded mbarrier wait (≈2 s), also gives up when another role raised the abort flag
__device__ __forceinline__ bool wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t it = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 63u) == 0u) {
      if (*abort_flag != 0) return false;
      if (globaltimer_ns() - t0 > 2000000000ull) return false;
    }
  }
}

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& mt, int& nt) {
  const int per_group = GROUP_M * num_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int gsize = min(num_m - first_m, GROUP_M);
  const int in_group = tile - group * per_group;
  mt = first_m + in_group % gsize;
  nt = in_group / gsize;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles want 1024-byte alignment
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + STAGES;          // [STAGES]
  uint64_t* tmem_full_bar = bars + 2 * STAGES;  // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2; // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full_bar[a], 1); mbar_init(&tmem_empty_bar[a], 4); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {  // one warp owns TMEM allocation and release
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mt, nt; tile_coords(tile, num_m, num_n, mt, nt);
        const int m0 = mt * BM, n0 = nt * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag)) {
            if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_EMPTY); }
            ok = false; break;
          }
          mbar_expect_tx(&full_bar[stage], A_STAGE_BYTES + B_STAGE_BYTES);
          uint8_t* sa = smem_a + stage * A_STAGE_BYTES;
          uint8_t* sb = smem_b + stage * B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);  // box {64 k, 128 m}
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)  // box {64 m, 64 k}, 8 KB each
              tma_load_2d(sa + j * 8192, &tmap_a, &full_bar[stage], m0 + j * 64, k0);
          }
          if (!p.b_mn) {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0);  // box {64 k, 256 n}
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[stage], n0 + j * 64, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(BM, BN, p.is_bf16 != 0, p.a_mn != 0, p.b_mn != 0);
      int stage = 0; uint32_t phase = 0; bool ok = true;
      int acc = 0; uint32_t acc_phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!wait_bounded(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag)) {
          if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_EMPTY); }
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_bounded(&full_bar[stage], phase, abort_flag)) {
            if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMA); }
            ok = false; break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem_a + stage * A_STAGE_BYTES);
          const uint32_t sb = smem_u32(smem_b + stage * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major : rows of 128 B, 8-row swizzle atoms 1024 B apart (SBO); a K step of 16 elements = +32 B
            // MN-major: 64-element (128 B) runs along M/N, K rows 128 B apart, 8-row atoms 1024 B apart (SBO),
            //           next 64-wide M/N block 8192 B further (LBO); a K step of 16 rows = +2048 B
            const uint64_t da = p.a_mn ? make_smem_desc(sa + k * 2048, 8192, 1024, 2)
                                       : make_smem_desc(sa + k * 32, 16, 1024, 2);
            const uint64_t db = p.b_mn ? make_smem_desc(sb + k * 2048, 8192, 1024, 2)
                                       : make_smem_desc(sb + k * 32, 16, 1024, 2);
            umma_f16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0; uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int mt, nt; tile_coords(tile, num_m, num_n, mt, nt);
      const int m0 = mt * BM, n0 = nt * BN;
      bool ok = wait_bounded(&tmem_full_bar[acc], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0 && *abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_FULL); }
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row < p.M && col < p.N) {
          if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col;
            if (col + 32 <= p.N) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 v = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                                       __uint_as_float(r[i + 3]));
                if (p.accumulate) {
                  const float4 o = *reinterpret_cast<const float4*>(dst + i);
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *reinterpret_cast<float4*>(dst + i) = v;
              }
            } else {
              for (int i = 0; i < 32 && col + i < p.N; ++i)
                dst[i] = __uint_as_float(r[i]) + (p.accumulate ? dst[i] : 0.f);
            }
          } else if (p.is_bf16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col;
            if (col + 32 <= p.N) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[i + j]);
                if (p.accumulate) {
                  const uint4 o = *reinterpret_cast<const uint4*>(dst + i);
                  const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) { const float2 t = unpack_bf16x2(ow[j]); f[2 * j] += t.x; f[2 * j + 1] += t.y; }
                }
                uint4 v = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                                     pack_bf16x2(f[6], f[7]));
                *reinterpret_cast<uint4*>(dst + i) = v;
              }
            } else {
              for (int i = 0; i < 32 && col + i < p.N; ++i)
                dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]) + (p.accumulate ? __bfloat162float(dst[i]) : 0.f));
            }
          } else {
            __half* dst = reinterpret_cast<__half*>(p.C) + (long long)row * p.ldc + col;
            for (int i = 0; i < 32 && col + i < p.N; ++i)
              dst[i] = __float2half_rn(__uint_as_float(r[i]) + (p.accumulate ? __half2float(dst[i]) : 0.f));
          }
        }
      }
      // accumulator buffer may be overwritten by the MMA warp now
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
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
  const CUtensorMapDataType dt = dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap ta, tb_;
  int rc;
  if (!a_mn) rc = tbh::make_tmap_2d(&ta, A, dt, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, BM, BK, 3);
  else       rc = tbh::make_tmap_2d(&ta, A, dt, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, 64, 64, 3);
  if (rc) return rc;
  if (!b_mn) rc = tbh::make_tmap_2d(&tb_, B, dt, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, BN, BK, 3);
  else       rc = tbh::make_tmap_2d(&tb_, B, dt, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, 64, 64, 3);
  if (rc) return rc;

  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    TB_CUDA_CHECK(cudaGetDevice(&dev));
    TB_CUDA_CHECK(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  TB_CUDA_CHECK(cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = tiles < sm_count ? tiles : sm_count;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn; p.out_fp32 = out_fp32; p.is_bf16 = dtype == 1;
  p.accumulate = accumulate; p.ldc = ldc; p.C = C; p.status = status;
  gemm_tcgen05_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, tb_, p);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
