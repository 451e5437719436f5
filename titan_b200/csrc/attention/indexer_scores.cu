// Lightning-indexer scores with the query operand resident in shared memory.
//
//   scores[s, t] = sum_h w[s, h] * relu(q[s, h, :] . k[t, :])        head dim 128, bf16, H a power of two (16 .. 256)
//   for every key t < (pos_offset + s + 1) / ratio  (ratio 1: causal tokens; ratio r: compressed keys of r tokens)
//
// The contraction is only 128 deep, so a generic tiled GEMM reloads 96 KB of operands for 0.9 us of tensor work per
// 128 x 256 tile and is bound by L2 -> SM traffic.  Here a CTA keeps one block of 256 (query, head) rows (64 KB: four
// queries of 64 heads) in shared memory and streams key tiles of 128 rows (32 KB) past it: a third of the traffic.
//
//   warp 0      TMA producer: the query block once per block, then key tiles through a 4-stage ring
//   warp 1      MMA issuer: S^T [128 keys x 256 (query, head)] = K_tile * Q_block^T into one of two accumulators
//   warps 2..5  epilogue: one key per thread (TMEM lane); the head sum of each query runs inside the thread
//               (relu, weight, add: no exchange between lanes), 128 consecutive keys are stored per query row
//
// Key tiles entirely in the causal future of the block's last query are never loaded.  Entries in the future of a
// query inside a computed tile are written but meaningless: consumers apply the same visibility rule.
// Every wait is bounded; a failure sets the status word and all roles drain to the common exit.
//
// Forward scoring of the reference's lightning indexer (torchtitan_npu/models/deepseek_v32/model.py:22-75,
// converters/kernels/dsa.py:60-130).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int D = 128;
constexpr int BKEYS = 128;
constexpr int BQH = 256;                 // (query, head) rows per block = N of the MMA
constexpr int STAGES = 4;
constexpr int A_BOX = BKEYS * 128;       // [128 keys x 64 d] bf16 = 16 KB
constexpr int A_STAGE = 2 * A_BOX;       // 32 KB
constexpr int B_BOX = BQH * 128;         // [256 rows x 64 d] = 32 KB
constexpr int NTHREADS = 192;
constexpr uint32_t TMEM_COLS = 512;      // two accumulators of 256 columns

struct IdxParams {
  const float* w;
  float* scores;
  long long ld;
  int S, H, T;
  int pos_offset, ratio;
  int* status;
};

struct __align__(8) Bars {
  uint64_t a_full[STAGES], a_empty[STAGES];
  uint64_t b_full, b_empty;
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_slot;
  int abort_flag;
};

__device__ __forceinline__ void fail(Bars* b, int* status, int code) {
  if (b->abort_flag == 0) {
    b->abort_flag = 1;
    if (status) atomicExch(status, code);
  }
}

__global__ void __launch_bounds__(NTHREADS, 1) indexer_scores_kernel(const __grid_constant__ CUtensorMap tm_k,
                                                                     const __grid_constant__ CUtensorMap tm_q,
                                                                     const IdxParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                               // STAGES x 32 KB
  uint8_t* sB = sA + STAGES * A_STAGE;              // 2 x 32 KB
  float* wst = reinterpret_cast<float*>(sB + 2 * B_BOX);   // 2 x 256 weights (alternating blocks)
  Bars* bars = reinterpret_cast<Bars*>(wst + 2 * BQH);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int N = p.S * p.H;
  const int nblocks = (N + BQH - 1) / BQH;
  const int hshift = 31 - __clz(p.H);

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&bars->a_full[i], 1); mbar_init(&bars->a_empty[i], 1); }
    mbar_init(&bars->b_full, 1); mbar_init(&bars->b_empty, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->acc_full[i], 1); mbar_init(&bars->acc_empty[i], 4); }
    bars->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_q);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  volatile int* abort_flag = &bars->abort_flag;

  // key tiles a block of (query, head) rows needs: up to the last visible key of its last query
  auto key_tiles = [&](int nb) {
    const int last_query = (min(nb * BQH + BQH, N) - 1) >> hshift;
    const int visible = min(p.T, (p.pos_offset + last_query + 1) / p.ratio);
    return (visible + BKEYS - 1) / BKEYS;
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0, bphase = 0;
      bool ok = true;
      for (int nb = blockIdx.x; nb < nblocks && ok; nb += gridDim.x) {
        if (!mbar_wait(&bars->b_empty, bphase ^ 1, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_EMPTY); break; }
        mbar_expect_tx(&bars->b_full, 2 * B_BOX);
        tma_load_2d(sB, &tm_q, &bars->b_full, 0, nb * BQH);
        tma_load_2d(sB + B_BOX, &tm_q, &bars->b_full, 64, nb * BQH);
        bphase ^= 1;
        const int mt = key_tiles(nb);
        for (int m = 0; m < mt; ++m) {
          if (!mbar_wait(&bars->a_empty[stage], phase ^ 1, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_EMPTY); ok = false; break; }
          mbar_expect_tx(&bars->a_full[stage], A_STAGE);
          tma_load_2d(sA + stage * A_STAGE, &tm_k, &bars->a_full[stage], 0, m * BKEYS);
          tma_load_2d(sA + stage * A_STAGE + A_BOX, &tm_k, &bars->a_full[stage], 64, m * BKEYS);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(BKEYS, BQH, true, false, false);
      const uint64_t da0 = make_smem_desc(smem_u32(sA), 16, 1024, 2);
      const uint64_t db0 = make_smem_desc(smem_u32(sB), 16, 1024, 2);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
      int stage = 0; uint32_t phase = 0, bphase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int nb = blockIdx.x; nb < nblocks && ok; nb += gridDim.x) {
        if (!mbar_wait(&bars->b_full, bphase, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_TMA); break; }
        bphase ^= 1;
        const int mt = key_tiles(nb);
        for (int m = 0; m < mt; ++m) {
          if (!mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_TMEM_EMPTY); ok = false; break; }
          if (!mbar_wait(&bars->a_full[stage], phase, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_TMA); ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem + acc * BQH;
          const uint32_t a_lo = a_lo0 + (uint32_t)stage * (A_STAGE >> 4);
#pragma unroll
          for (int c = 0; c < 2; ++c)        // 64-wide halves of the head dim
#pragma unroll
            for (int k = 0; k < 4; ++k)      // K steps of 16 elements (32 B)
              umma_f16_lohi(d, a_lo + c * (A_BOX >> 4) + k * 2, a_hi, b_lo0 + c * (B_BOX >> 4) + k * 2, b_hi, idesc,
                            (c | k) ? 1u : 0u);
          umma_commit(&bars->a_empty[stage]);
          umma_commit(&bars->acc_full[acc]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        umma_commit(&bars->b_empty);   // arrives when every product that read this query block has finished
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int q4 = warp & 3;                          // TMEM lane quarter this warp may read
    const int et = (warp - 2) * 32 + lane;            // 0..127 among the epilogue threads
    const int row_in_tile = q4 * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(q4 * 32) << 16);
    const int hmask = p.H - 1;
    int acc = 0; uint32_t acc_phase = 0;
    int wbuf = 0;
    bool ok = true;
    for (int nb = blockIdx.x; nb < nblocks && ok; nb += gridDim.x) {
      const int n0 = nb * BQH;
      float* wt = wst + wbuf * BQH;                   // alternating buffers: no wait for the previous block's readers
      for (int i = et; i < BQH; i += 128) wt[i] = (n0 + i) < N ? p.w[n0 + i] : 0.f;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int mt = key_tiles(nb);
      for (int m = 0; m < mt; ++m) {
        if (!mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_TMEM_FULL); ok = false; break; }
        tc_fence_after();
        const int key = m * BKEYS + row_in_tile;
        const uint32_t taddr = lane_base + acc * BQH;
        if (p.H >= 32) {
          // a query's heads end on 32-column chunk boundaries: four independent accumulators, weights as 128-bit
          // shared loads, the next chunk's tcgen05.ld in flight while this one is summed
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
          uint32_t r[2][32];
          tmem_ld_32x32(taddr, r[0]);
#pragma unroll
          for (int c = 0; c < BQH / 32; ++c) {
            tmem_ld_wait();
            if (c + 1 < BQH / 32) tmem_ld_32x32(taddr + (c + 1) * 32, r[(c + 1) & 1]);
            const float4* w4 = reinterpret_cast<const float4*>(wt + c * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 w = w4[i];
              s0 = fmaf(fmaxf(__uint_as_float(r[c & 1][4 * i + 0]), 0.f), w.x, s0);
              s1 = fmaf(fmaxf(__uint_as_float(r[c & 1][4 * i + 1]), 0.f), w.y, s1);
              s2 = fmaf(fmaxf(__uint_as_float(r[c & 1][4 * i + 2]), 0.f), w.z, s2);
              s3 = fmaf(fmaxf(__uint_as_float(r[c & 1][4 * i + 3]), 0.f), w.w, s3);
            }
            if ((((c + 1) * 32) & hmask) == 0) {      // last head of a query
              const int query = (n0 + c * 32) >> hshift;
              if (key < p.T && query < p.S) p.scores[(long long)query * p.ld + key] = (s0 + s1) + (s2 + s3);
              s0 = s1 = s2 = s3 = 0.f;
            }
          }
        } else {
          float sum = 0.f;
#pragma unroll 1
          for (int c = 0; c < BQH / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              sum = fmaf(fmaxf(__uint_as_float(r[i]), 0.f), wt[c * 32 + i], sum);
              if (((c * 32 + i + 1) & hmask) == 0) {
                const int query = (n0 + c * 32 + i) >> hshift;
                if (key < p.T && query < p.S) p.scores[(long long)query * p.ld + key] = sum;
                sum = 0.f;
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      wbuf ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}
}  // namespace

// q: [S*H, 128] bf16 (row = query*H + head; H a power of two, 16 .. 256), k: [T, 128] bf16, w: [S*H] fp32,
// scores: [S, ld] fp32.  See the header for the visibility rule.
TB_API int tb_indexer_scores_resident(const void* q, const void* k, const float* w, float* scores, int S, int H, int T,
                                      int head_dim, long long ld, int pos_offset, int ratio, int* status,
                                      cudaStream_t st) {
  if (S <= 0 || T <= 0) return 0;
  if (head_dim != D || ratio < 1 || H < 16 || H > BQH || (H & (H - 1)) != 0 || ld < T) return TB_ERR_ARG;
  if ((long long)S * H > 0x7fffffffLL) return TB_ERR_ARG;
  CUtensorMap tk, tq;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (int rc = tbh::make_tmap_2d(&tk, k, bf, 2, (uint64_t)T, D, D * 2, BKEYS, 64, 3)) return rc;
  if (int rc = tbh::make_tmap_2d(&tq, q, bf, 2, (uint64_t)S * H, D, D * 2, BQH, 64, 3)) return rc;
  IdxParams p{};
  p.w = w; p.scores = scores; p.ld = ld;
  p.S = S; p.H = H; p.T = T; p.pos_offset = pos_offset; p.ratio = ratio; p.status = status;
  const int smem = STAGES * A_STAGE + 2 * B_BOX + 2 * BQH * 4 + (int)sizeof(Bars) + 1024;
  TB_CUDA_CHECK(cudaFuncSetAttribute(indexer_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int nblocks = (int)(((long long)S * H + BQH - 1) / BQH);
  indexer_scores_kernel<<<nblocks < sms ? nblocks : sms, NTHREADS, smem, st>>>(tk, tq, p);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
