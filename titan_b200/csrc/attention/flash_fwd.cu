// Causal flash attention forward for sm_100a: tcgen05 MMAs with accumulators in tensor memory, TMA-fed operands.
//
//   Q [B, S, H, D], K / V [B, S, Hkv, D] (bf16, D = 128, H a multiple of Hkv), O [B, S, H, D], LSE [B, H, S] fp32.
//
// One CTA per (batch, head, 128-query block); it walks the key blocks 0 .. diagonal (128 keys each):
//   warp 0      TMA producer: Q once, then K_j and V_j through two-stage rings (128B-swizzled tiles)
//   warp 1      MMA issuer (one thread): S_j = Q K_j^T  (M128 N128 K128, both operands K-major)
//                                        PV_j = P_j V_j (A = P_j from shared memory, B = V_j MN-major)
//               S_{j+1} is issued before PV_j so the tensor cores work while the softmax warps handle block j
//   warps 2..9  softmax, TWO threads per query row (TMEM lane = row; warps w and w+4 share a lane quarter and take
//               64 of the 128 columns each): one read of S_j from tensor memory into registers, row maximum
//               (halves exchanged through shared memory), exp2 / row sum / bf16 P_j into the swizzled A-operand
//               layout, then fold PV_{j-1} into the running output kept in REGISTERS (64 fp32 per thread):
//               O <- (O + PV_{j-1}) * 2^(m_{j-1}-m_j)
// Tensor memory: S double-buffered (2 x 128 columns) + PV double-buffered (2 x 128 columns) = all 512 columns.
// Shared memory: Q 32 KB + K 2 x 32 KB + V 2 x 32 KB + P 2 x 32 KB = 224 KB, + 2 KB exchange area and barriers.
//
// Every wait is bounded (mbar_wait gives up after 2^22 polls): on expiry the role records a status code, raises the
// CTA-wide abort flag, and all roles drain to the common exit where the tensor memory is freed.
//
// Semantics: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True) — the
// reference's fused attention op (K7: npu_fusion_attention, BSND layout).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int D = 128;        // head dim
constexpr int BQ = 128;       // query rows per CTA
constexpr int BK = 128;       // keys per block
constexpr int TILE = 32768;   // bytes of a [128 x 128] bf16 tile (two 16 KB boxes of 64 columns)
constexpr int NTHREADS = 320;  // TMA warp, MMA warp, 8 softmax warps
constexpr uint32_t TMEM_COLS = 512;

struct FaParams {
  int B, S, H, Hkv;
  float scale_log2;  // softmax scale * log2(e)
  __nv_bfloat16* O;
  float* LSE;
  const int* seq_start;  // [B * S] first position of each token's document (packed sequences), or null
  int* status;
};

struct __align__(8) Bars {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], s_empty[2], p_ready[2], o_full[2], o_empty[2];
  uint32_t tmem_slot;
  int abort_flag;
  float xchg[2][2][BQ];  // [parity][column half][row]: row maxima (and, at the end, row sums) of the two halves
};

__device__ __forceinline__ void fail(Bars* b, int* status, int code) {
  if (b->abort_flag == 0) {
    b->abort_flag = 1;
    if (status) atomicExch(status, code);
  }
}

// VARLEN: packed documents (`seq_start` given).  The dense instance carries none of the extra masking code.
template <bool VARLEN>
__global__ void __launch_bounds__(NTHREADS, 1) flash_fwd_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                const __grid_constant__ CUtensorMap tm_k,
                                                                const __grid_constant__ CUtensorMap tm_v,
                                                                const FaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // The tiles need 1024-byte alignment and there is no room for alignment slack (224 KB of tiles + barriers +
  // exchange area): the dynamic window of a kernel without static shared memory starts aligned; otherwise refuse.
  if ((smem_u32(smem_raw) & 1023u) != 0u) {
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, TB_ERR_ARG);
    return;
  }
  uint8_t* smem = smem_raw;
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE;          // 2 stages
  uint8_t* sV = smem + 3 * TILE;      // 2 stages
  uint8_t* sP = smem + 5 * TILE;      // 2 buffers
  Bars* bars = reinterpret_cast<Bars*>(smem + 7 * TILE);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy tiles (late query blocks) first
  const int nq = p.S / BQ;
  const int qb = nq - 1 - (int)blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q_row0 = b * p.S + qb * BQ;
  // causal: key blocks j0 .. qb.  With packed documents the block's first query belongs to the earliest document of
  // the block (documents start at non-decreasing positions), so no row needs a key block before that document.
  const int j0 = VARLEN ? p.seq_start[q_row0] / BK : 0;
  const int nblk = qb + 1 - j0;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], 1); mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1); mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1); mbar_init(&bars->s_empty[i], 8);
      mbar_init(&bars->p_ready[i], 8);
      mbar_init(&bars->o_full[i], 1); mbar_init(&bars->o_empty[i], 8);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
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

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, TILE);
      tma_load_2d(sQ, &tm_q, &bars->q_full, h * D, q_row0);
      tma_load_2d(sQ + 16384, &tm_q, &bars->q_full, h * D + 64, q_row0);
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int k_row0 = b * p.S + (j0 + j) * BK;
        if (!mbar_wait(&bars->k_empty[st], ph ^ 1, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_EMPTY); break; }
        mbar_expect_tx(&bars->k_full[st], TILE);
        tma_load_2d(sK + st * TILE, &tm_k, &bars->k_full[st], hk * D, k_row0);
        tma_load_2d(sK + st * TILE + 16384, &tm_k, &bars->k_full[st], hk * D + 64, k_row0);
        if (!mbar_wait(&bars->v_empty[st], ph ^ 1, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_EMPTY); break; }
        mbar_expect_tx(&bars->v_full[st], TILE);
        // V is the MN-major B operand: per 64-key chunk two boxes of {64 d, 64 keys} (8 KB each)
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int dbx = 0; dbx < 2; ++dbx)
            tma_load_2d(sV + st * TILE + c * 16384 + dbx * 8192, &tm_v, &bars->v_full[st], hk * D + dbx * 64,
                        k_row0 + c * 64);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_f16(BQ, BK, true, false, false);
      const uint32_t idesc_pv = make_idesc_f16(BQ, D, true, false, true);
      const uint32_t aQ = smem_u32(sQ);
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag);
      if (!ok) fail(bars, p.status, TB_ERR_WAIT_TMA);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bars->k_full[st], ph, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_TMA); return false; }
        if (!mbar_wait(&bars->s_empty[st], ph ^ 1, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_TMEM_EMPTY); return false; }
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + st * TILE);
#pragma unroll
        for (int c = 0; c < 2; ++c)        // 64-wide boxes of the head dim
#pragma unroll
          for (int k = 0; k < 4; ++k)      // K steps of 16 elements (32 B)
            umma_f16(tmem + st * BK, make_smem_desc(aQ + c * 16384 + k * 32, 16, 1024, 2),
                     make_smem_desc(aK + c * 16384 + k * 32, 16, 1024, 2), idesc_s, (c | k) ? 1u : 0u);
        umma_commit(&bars->k_empty[st]);
        umma_commit(&bars->s_full[st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) ok = issue_s(j + 1);
        if (!ok) break;
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bars->p_ready[st], ph, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_TMEM_FULL); break; }
        if (!mbar_wait(&bars->v_full[st], ph, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_TMA); break; }
        if (!mbar_wait(&bars->o_empty[st], ph ^ 1, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_TMEM_EMPTY); break; }
        tc_fence_after();
        const uint32_t aP = smem_u32(sP + st * TILE), aV = smem_u32(sV + st * TILE);
#pragma unroll
        for (int c = 0; c < 2; ++c)        // 64-key chunks
#pragma unroll
          for (int k = 0; k < 4; ++k)      // 16 keys per step
            umma_f16(tmem + 2 * BK + st * D, make_smem_desc(aP + c * 16384 + k * 32, 16, 1024, 2),
                     make_smem_desc(aV + c * 16384 + k * 2048, 8192, 1024, 2), idesc_pv, (c | k) ? 1u : 0u);
        umma_commit(&bars->v_empty[st]);
        umma_commit(&bars->o_full[st]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + output (warps 2..9)
    constexpr int HC = BK / 2;            // columns per thread
    const int quarter = warp & 3;         // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;     // which 64 columns of S / PV / O
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const int pair_bar = 2 + quarter;     // named barrier of the two warps that share this lane quarter
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory"); };
    auto ex2 = [](float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; };
    float m_run = -INFINITY, l_run = 0.f;
    float o[HC];
#pragma unroll
    for (int i = 0; i < HC; ++i) o[i] = 0.f;
    // A thread that gives up (a bounded wait ran out) must not leave its partner alone at the pair barrier: it keeps
    // walking to the next exchange, publishes NaN there, and both leave together right after that barrier.
    bool ok = true;
    // keys before the start of this row's document are masked: key column c of block j is allowed from `lo` on
    const int row_start = VARLEN ? p.seq_start[q_row0 + row] : 0;
    for (int j = 0; j < nblk; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (ok && !mbar_wait(&bars->s_full[st], ph, abort_flag)) { fail(bars, p.status, TB_ERR_WAIT_TMEM_FULL); ok = false; }
      tc_fence_after();
      const uint32_t s_addr = lane_base + st * BK + half * HC;
      const bool diag = j == nblk - 1;
      const int lo = VARLEN ? row_start - (j0 + j) * BK : 0;   // first allowed column of this block (<= 0: all)
      const bool edge = diag || (VARLEN && lo > 0);
      uint32_t r[2][32];
      float mx = -INFINITY;
      if (ok) {
        tmem_ld_32x32(s_addr, r[0]);
        tmem_ld_32x32(s_addr + 32, r[1]);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (!edge || ((!diag || half * HC + c * 32 + i <= row) && (!VARLEN || half * HC + c * 32 + i >= lo)))
              mx = fmaxf(mx, __uint_as_float(r[c][i]));
      }
      bars->xchg[st][half][row] = ok ? mx : NAN;
      pair_sync();
      const float other = bars->xchg[st][half ^ 1][row];
      if (!ok || other != other) { ok = false; break; }
      const float m_new = fmaxf(m_run, fmaxf(mx, other) * p.scale_log2);
      // a row whose document starts after this block has seen no key yet: keep its state untouched
      const float alpha = (VARLEN && m_new == -INFINITY) ? 1.f : ex2(m_run - m_new);
      // P = 2^(s' - m), row sum, bf16 into the swizzled K-major A-operand layout (this thread's 64 keys = one box)
      float sum = 0.f;
      const uint32_t prow = smem_u32(sP + st * TILE) + row * 128 + half * 16384;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = ex2(fmaf(__uint_as_float(r[c][2 * i]), p.scale_log2, -m_new));
          float p1 = ex2(fmaf(__uint_as_float(r[c][2 * i + 1]), p.scale_log2, -m_new));
          if (edge) {
            const int col = half * HC + c * 32 + 2 * i;
            if ((diag && col > row) || (VARLEN && col < lo)) p0 = 0.f;
            if ((diag && col + 1 > row) || (VARLEN && col + 1 < lo)) p1 = 0.f;
          }
          sum += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t chunk = (uint32_t)(c * 4 + i) ^ (uint32_t)(row & 7);  // 128B swizzle
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + chunk * 16), "r"(pk[4 * i]),
                       "r"(pk[4 * i + 1]), "r"(pk[4 * i + 2]), "r"(pk[4 * i + 3])
                       : "memory");
        }
      }
      l_run = l_run * alpha + sum;
      m_run = m_new;
      tc_fence_before();
      fence_proxy_async();  // P was written by ordinary stores; the MMA reads it through the async proxy
      __syncwarp();
      if (lane == 0) { mbar_arrive(&bars->s_empty[st]); mbar_arrive(&bars->p_ready[st]); }
      if (j >= 1) {
        const int ps = (j - 1) & 1;
        if (!mbar_wait(&bars->o_full[ps], ((j - 1) >> 1) & 1, abort_flag)) {
          fail(bars, p.status, TB_ERR_WAIT_TMEM_FULL);
          ok = false;
          continue;  // to the next exchange (or the final one), where the pair leaves together
        }
        tc_fence_after();
        const uint32_t o_addr = lane_base + 2 * BK + ps * D + half * HC;
        const bool rescale = alpha != 1.f;  // the running maximum moved
#pragma unroll
        for (int c = 0; c < HC / 32; ++c) {
          uint32_t pv[32];
          tmem_ld_32x32(o_addr + c * 32, pv);
          tmem_ld_wait();
          if (rescale) {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(pv[i])) * alpha;
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(pv[i]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->o_empty[ps]);
      }
    }
    {
      // final exchange: partial row sums (NaN = this half gave up)
      const int xs = nblk & 1;
      const int ps = (nblk - 1) & 1;
      if (ok && !mbar_wait(&bars->o_full[ps], ((nblk - 1) >> 1) & 1, abort_flag)) {
        fail(bars, p.status, TB_ERR_WAIT_TMEM_FULL);
        ok = false;
      }
      bars->xchg[xs][half][row] = ok ? l_run : NAN;
      pair_sync();
      const float l_other = bars->xchg[xs][half ^ 1][row];
      if (ok && l_other == l_other) {
        tc_fence_after();
        const float l_tot = l_run + l_other;
        const uint32_t o_addr = lane_base + 2 * BK + ps * D + half * HC;
        const float inv = 1.f / l_tot;
        __nv_bfloat16* dst = p.O + ((size_t)(q_row0 + row) * p.H + h) * D + half * HC;
#pragma unroll
        for (int c = 0; c < HC / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(o_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int col = c * 32 + i * 8 + e * 2;
              w[e] = pack_bf16x2((o[col] + __uint_as_float(r[i * 8 + e * 2])) * inv,
                                 (o[col + 1] + __uint_as_float(r[i * 8 + e * 2 + 1])) * inv);
            }
            *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = v;
          }
        }
        if (p.LSE != nullptr && half == 0)
          p.LSE[((size_t)b * p.H + h) * p.S + qb * BQ + row] = (m_run + log2f(l_tot)) * 0.6931471805599453f;
        tc_fence_before();
      }
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}
}  // namespace

// q: [B, S, H, 128] bf16, k / v: [B, S, Hkv, 128] bf16 (contiguous), out: [B, S, H, 128] bf16, lse: [B, H, S] fp32 or
// nullptr; seq_start: [B * S] int32 (position of the first token of each token's document, non-decreasing along a
// sequence) for packed documents, or nullptr.  S must be a multiple of 128.
TB_API int tb_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* seq_start,
                             int B, int S, int H, int Hkv, int head_dim, float scale, int* status, cudaStream_t st) {
  if (B <= 0 || S <= 0) return 0;
  if (head_dim != D || S % BQ != 0 || Hkv < 1 || H % Hkv != 0 || (long long)B * S > 0x7fffffffLL) return TB_ERR_ARG;
  CUtensorMap tq, tk, tv;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (int rc = tbh::make_tmap_2d(&tq, q, bf, 2, (uint64_t)B * S, (uint64_t)H * D, (uint64_t)H * D * 2, BQ, 64, 3)) return rc;
  if (int rc = tbh::make_tmap_2d(&tk, k, bf, 2, (uint64_t)B * S, (uint64_t)Hkv * D, (uint64_t)Hkv * D * 2, BK, 64, 3)) return rc;
  if (int rc = tbh::make_tmap_2d(&tv, v, bf, 2, (uint64_t)B * S, (uint64_t)Hkv * D, (uint64_t)Hkv * D * 2, 64, 64, 3)) return rc;
  FaParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.O = (__nv_bfloat16*)out; p.LSE = lse; p.seq_start = seq_start; p.status = status;
  const size_t smem = 7 * TILE + sizeof(Bars);
  if (seq_start != nullptr) {
    TB_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  } else {
    TB_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  dim3 grid(S / BQ, H, B);
  if (seq_start != nullptr) flash_fwd_kernel<true><<<grid, NTHREADS, smem, st>>>(tq, tk, tv, p);
  else flash_fwd_kernel<false><<<grid, NTHREADS, smem, st>>>(tq, tk, tv, p);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
