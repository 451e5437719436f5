// Causal flash attention backward for sm_100a on tcgen05 tensor cores, with per-document masking for packed
// (variable-length) sequences.
//
//   Q, dO [B, S, H, D], K, V [B, S, Hkv, D] bf16 (D = 128, H a multiple of Hkv); LSE, DELTA [B, H, S] fp32
//   (LSE natural log from the forward, DELTA = rowsum(dO * O)); seq_start [B * S] int32 or null: the position (inside
//   the sequence) of the first token of each token's document.  A query at position s sees the keys
//   seq_start[s] .. s.
//   Outputs: dK, dV [B, S, Hkv, D] bf16 (written), dQ32 [B, S, H, D] fp32 (ACCUMULATED: zero it before the launch).
//
// One CTA owns one (batch, kv head, block of 128 keys) and walks every (query head of the group, query block at or
// after the key block).  Keys sit on the M axis (TMEM lane = key), so the softmax recomputation needs no row
// reductions: a thread owns one key and a range of queries.
//
//   S^T  [keys x q] = K  * Q^T          A = K tile K-major,   B = Q tile K-major
//   dP^T [keys x q] = V  * dO^T         A = V tile K-major,   B = dO tile K-major
//   P^T = exp(S^T * scale - lse[q]),  dS^T = P^T * (dP^T - delta[q]) * scale      (threads; masks applied here)
//   dV [keys x D] += P^T  * dO          A = P^T  K-major (shared memory),   B = dO tile MN-major
//   dK [keys x D] += dS^T * Q           A = dS^T K-major,                   B = Q tile MN-major
//   dQ [q x D]     = dS   * K           A = dS^T read MN-major (M = queries), B = K tile MN-major
//
// dK and dV stay in tensor memory over the whole walk and are written once (no atomics, GQA heads summed in place);
// the dQ partial of each (query block, key block) pair is added to the fp32 buffer with 16-byte vector reductions.
// Tensor memory: S^T / dQ (shared columns), dP^T, dK, dV = 4 x 128 columns.
// Shared memory: K, V, Q, dO, P^T, dS^T tiles of 32 KB each.
//
// Every wait is bounded; a failure sets the status word and the CTA drains to the common exit.
//
// Semantics: the gradient of torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True,
// enable_gqa=True), per document when `seq_start` is given — the reference's fused attention gradient
// (K7 `npu_fusion_attention_grad`, causal / TND packed layout, torchtitan_npu/models/common/npu_varlen_attention.py:42-97).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int D = 128;
constexpr int BLK = 128;           // queries per block = keys per block
constexpr int TILE = 32768;        // [128 x 128] bf16 as two [128 rows x 64 columns] boxes
constexpr int BOX = 16384;
constexpr int NTHREADS = 256;
constexpr uint32_t TMEM_COLS = 512;

struct FbParams {
  int B, S, H, Hkv;
  float scale, scale_log2;
  const float* lse;
  const float* delta;
  const int* seq_start;
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  float* dQ;
  int* status;
};

struct __align__(16) Ctl {
  float lse2[BLK], delta[BLK];   // 16-byte aligned: read four at a time
  int qstart[BLK];
  uint64_t kv_bar, q_bar, mma_bar;
  uint32_t tmem_slot;
  int abort_flag;
};

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float4 ld_shared_f4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// VARLEN: packed documents (`seq_start` given); the dense instance carries no document-mask code.
template <bool VARLEN>
__global__ void __launch_bounds__(NTHREADS, 1) flash_bwd_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                const __grid_constant__ CUtensorMap tm_do,
                                                                const __grid_constant__ CUtensorMap tm_k,
                                                                const __grid_constant__ CUtensorMap tm_v,
                                                                const FbParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE;
  uint8_t* sQ = smem + 2 * TILE;
  uint8_t* sDO = smem + 3 * TILE;
  uint8_t* sP = smem + 4 * TILE;
  uint8_t* sDS = smem + 5 * TILE;
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + 6 * TILE);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nblk = p.S / BLK;
  const int j = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int gsz = p.H / p.Hkv;
  const int k_row0 = b * p.S + j * BLK;

  if (tid == 0) {
    mbar_init(&ctl->kv_bar, 1);
    mbar_init(&ctl->q_bar, 1);
    mbar_init(&ctl->mma_bar, 1);
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_do); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_slot;
  const uint32_t tmem_s = tmem, tmem_dp = tmem + 128, tmem_dk = tmem + 256, tmem_dv = tmem + 384;
  volatile int* abort_flag = &ctl->abort_flag;
  const int quarter = warp & 3, half = warp >> 2;
  const int r = quarter * 32 + lane;                       // TMEM lane of this thread
  const uint32_t lane_off = ((uint32_t)(quarter * 32)) << 16;

  // the query blocks this key block takes part in: i = j .. i_end - 1 (documents start at non-decreasing positions,
  // so the first block whose first query's document starts after the last key of this block ends the walk)
  int i_end = nblk;
  if (VARLEN) {
    for (int i = j + 1; i < nblk; ++i)
      if (p.seq_start[(long long)b * p.S + i * BLK] > j * BLK + BLK - 1) { i_end = i; break; }
  }
  const int per_head = i_end - j;
  const int iters = per_head * gsz;

  auto load_q = [&](int it) {   // thread 0: Q and dO tiles of iteration `it`
    const int h = hk * gsz + it / per_head, i = j + it % per_head;
    const int q_row0 = b * p.S + i * BLK;
    mbar_expect_tx(&ctl->q_bar, 2 * TILE);
    tma_load_2d(sQ, &tm_q, &ctl->q_bar, h * D, q_row0);
    tma_load_2d(sQ + BOX, &tm_q, &ctl->q_bar, h * D + 64, q_row0);
    tma_load_2d(sDO, &tm_do, &ctl->q_bar, h * D, q_row0);
    tma_load_2d(sDO + BOX, &tm_do, &ctl->q_bar, h * D + 64, q_row0);
  };
  auto load_stats = [&](int it) {   // threads 0..127: per-query statistics of iteration `it`
    const int h = hk * gsz + it / per_head, i = j + it % per_head;
    const long long o = ((long long)b * p.H + h) * p.S + i * BLK + tid;
    ctl->lse2[tid] = p.lse[o] * 1.4426950408889634f;
    ctl->delta[tid] = p.delta[o];
    if (VARLEN) ctl->qstart[tid] = p.seq_start[(long long)b * p.S + i * BLK + tid];
  };

  if (tid == 0) {
    mbar_expect_tx(&ctl->kv_bar, 2 * TILE);
    tma_load_2d(sK, &tm_k, &ctl->kv_bar, hk * D, k_row0);
    tma_load_2d(sK + BOX, &tm_k, &ctl->kv_bar, hk * D + 64, k_row0);
    tma_load_2d(sV, &tm_v, &ctl->kv_bar, hk * D, k_row0);
    tma_load_2d(sV + BOX, &tm_v, &ctl->kv_bar, hk * D + 64, k_row0);
    load_q(0);
  }
  if (tid < BLK) load_stats(0);
  if (!mbar_wait(&ctl->kv_bar, 0, abort_flag)) {
    if (tid == 0 && *abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMA); }
  }
  __syncthreads();

  const uint32_t idesc_kk = make_idesc_f16(128, 128, true, false, false);   // both operands K-major
  const uint32_t idesc_kn = make_idesc_f16(128, 128, true, false, true);    // A K-major, B MN-major
  const uint32_t idesc_nn = make_idesc_f16(128, 128, true, true, true);     // both MN-major
  uint32_t q_phase = 0, mma_phase = 0;

  for (int it = 0; it < iters && *abort_flag == 0; ++it) {
    const int h = hk * gsz + it / per_head, i = j + it % per_head;
    if (!mbar_wait(&ctl->q_bar, q_phase, abort_flag)) {
      if (tid == 0 && *abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMA); }
    }
    q_phase ^= 1;
    if (*abort_flag) break;

    // ---- S^T = K Q^T, dP^T = V dO^T
    if (tid == 0) {
      tc_fence_after();
      const uint32_t ak = smem_u32(sK), av = smem_u32(sV), aq = smem_u32(sQ), ado = smem_u32(sDO);
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tmem_s, make_smem_desc(ak + c * BOX + k * 32, 16, 1024, 2),
                   make_smem_desc(aq + c * BOX + k * 32, 16, 1024, 2), idesc_kk, (c | k) ? 1u : 0u);
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tmem_dp, make_smem_desc(av + c * BOX + k * 32, 16, 1024, 2),
                   make_smem_desc(ado + c * BOX + k * 32, 16, 1024, 2), idesc_kk, (c | k) ? 1u : 0u);
      umma_commit(&ctl->mma_bar);
    }
    if (!mbar_wait(&ctl->mma_bar, mma_phase, abort_flag)) {
      if (tid == 0 && *abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_FULL); }
    }
    mma_phase ^= 1;
    tc_fence_after();
    __syncthreads();   // also: the statistics of this iteration are visible
    if (*abort_flag) break;

    // ---- P^T and dS^T: thread = (key r, 64 queries of its half), 32 queries per pass.  Masks only where they can
    //      bite: the causal one on the diagonal block, the document one when the batch is packed.
    {
      const int kpos = j * BLK + r;
      const int qpos0 = i * BLK;
      const bool diag = i == j;
#pragma unroll 1
      for (int pass = 0; pass < 2; ++pass) {
        const int c0 = half * 64 + pass * 32;          // first query column of this pass
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tmem_s + lane_off + c0, sv);
        tmem_ld_32x32(tmem_dp + lane_off + c0, dv);
        tmem_ld_wait();
        uint32_t pp[16], ds[16];
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {               // four queries per step: statistics read as float4
          const float4 l4 = ld_shared_f4(&ctl->lse2[c0 + 4 * e4]);
          const float4 d4 = ld_shared_f4(&ctl->delta[c0 + 4 * e4]);
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dl[4] = {d4.x, d4.y, d4.z, d4.w};
          float pv[4], dsv[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int qc = c0 + 4 * e4 + u;
            float pr = ex2_approx(fmaf(__uint_as_float(sv[4 * e4 + u]), p.scale_log2, -lv[u]));
            if (diag && qpos0 + qc < kpos) pr = 0.f;
            if (VARLEN && kpos < ctl->qstart[qc]) pr = 0.f;
            pv[u] = pr;
            dsv[u] = pr * (__uint_as_float(dv[4 * e4 + u]) - dl[u]) * p.scale;
          }
          pp[2 * e4] = pack_bf16x2(pv[0], pv[1]);
          pp[2 * e4 + 1] = pack_bf16x2(pv[2], pv[3]);
          ds[2 * e4] = pack_bf16x2(dsv[0], dsv[1]);
          ds[2 * e4 + 1] = pack_bf16x2(dsv[2], dsv[3]);
        }
        // row r of the [keys x queries] operand tile: box c0 / 64, 16-byte slots ((c0 % 64) / 8 + s) ^ (r & 7)
        const uint32_t rowoff = (uint32_t)(c0 >> 6) * BOX + (uint32_t)r * 128;
        const int slot0 = (c0 & 63) >> 3;
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) {
          const uint32_t o = rowoff + ((uint32_t)((slot0 + s4) ^ (r & 7)) << 4);
          st_shared_v4(smem_u32(sP) + o, pp[4 * s4], pp[4 * s4 + 1], pp[4 * s4 + 2], pp[4 * s4 + 3]);
          st_shared_v4(smem_u32(sDS) + o, ds[4 * s4], ds[4 * s4 + 1], ds[4 * s4 + 2], ds[4 * s4 + 3]);
        }
      }
      tc_fence_before();
    }
    fence_proxy_async();
    __syncthreads();

    // ---- dV += P^T dO, dK += dS^T Q, dQ = dS K
    if (tid == 0) {
      tc_fence_after();
      const uint32_t ak = smem_u32(sK), aq = smem_u32(sQ), ado = smem_u32(sDO), ap = smem_u32(sP), ads = smem_u32(sDS);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)   // 16 queries per step
        umma_f16(tmem_dv, make_smem_desc(ap + (kk >> 2) * BOX + (kk & 3) * 32, 16, 1024, 2),
                 make_smem_desc(ado + kk * 2048, BOX, 1024, 2), idesc_kn, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_f16(tmem_dk, make_smem_desc(ads + (kk >> 2) * BOX + (kk & 3) * 32, 16, 1024, 2),
                 make_smem_desc(aq + kk * 2048, BOX, 1024, 2), idesc_kn, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)   // 16 keys per step
        umma_f16(tmem_s, make_smem_desc(ads + kk * 2048, BOX, 1024, 2),
                 make_smem_desc(ak + kk * 2048, BOX, 1024, 2), idesc_nn, kk > 0 ? 1u : 0u);
      umma_commit(&ctl->mma_bar);
    }
    if (!mbar_wait(&ctl->mma_bar, mma_phase, abort_flag)) {
      if (tid == 0 && *abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_FULL); }
    }
    mma_phase ^= 1;
    tc_fence_after();
    __syncthreads();
    if (*abort_flag) break;

    // ---- the next iteration's tiles and statistics travel while dQ is written out
    if (it + 1 < iters) {
      if (tid == 0) load_q(it + 1);
      if (tid < BLK) load_stats(it + 1);
    }
    {
      float* dst = p.dQ + (((long long)b * p.S + i * BLK + r) * p.H + h) * D + half * 64;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_s + lane_off + half * 64 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; e += 4)
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c + e),
                       "f"(__uint_as_float(v[e])), "f"(__uint_as_float(v[e + 1])), "f"(__uint_as_float(v[e + 2])),
                       "f"(__uint_as_float(v[e + 3]))
                       : "memory");
      }
      tc_fence_before();
    }
    __syncthreads();   // S^T / dQ columns and the statistics are free for the next iteration
  }

  // ---- dK, dV of this key block (lane = key, two warp sets split the columns)
  if (*abort_flag == 0 && iters > 0) {
    tc_fence_after();
    const long long o = ((long long)(k_row0 + r) * p.Hkv + hk) * D + half * 64;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* dst = (which == 0 ? p.dK : p.dV) + o;
      const uint32_t src = (which == 0 ? tmem_dk : tmem_dv) + lane_off + half * 64;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(src + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(v[e]), __uint_as_float(v[e + 1]));
          w.y = pack_bf16x2(__uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
          w.z = pack_bf16x2(__uint_as_float(v[e + 4]), __uint_as_float(v[e + 5]));
          w.w = pack_bf16x2(__uint_as_float(v[e + 6]), __uint_as_float(v[e + 7]));
          *reinterpret_cast<uint4*>(dst + c + e) = w;
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}
}  // namespace

// q, dout [B, S, H, 128], k, v [B, S, Hkv, 128] bf16 contiguous; lse, delta [B, H, S] fp32; seq_start [B * S] int32 or
// null; dk, dv [B, S, Hkv, 128] bf16 (overwritten); dq32 [B, S, H, 128] fp32, zero-filled by the caller.
TB_API int tb_flash_attn_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                             const float* delta, const int* seq_start, void* dk, void* dv, float* dq32, int B, int S,
                             int H, int Hkv, int head_dim, float scale, int* status, cudaStream_t st) {
  if (B <= 0 || S <= 0) return 0;
  if (head_dim != D || S % BLK != 0 || Hkv < 1 || H % Hkv != 0 || (long long)B * S > 0x7fffffffLL) return TB_ERR_ARG;
  CUtensorMap tq, tdo, tk, tv;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint64_t rows = (uint64_t)B * S;
  if (int rc = tbh::make_tmap_2d(&tq, q, bf, 2, rows, (uint64_t)H * D, (uint64_t)H * D * 2, BLK, 64, 3)) return rc;
  if (int rc = tbh::make_tmap_2d(&tdo, dout, bf, 2, rows, (uint64_t)H * D, (uint64_t)H * D * 2, BLK, 64, 3)) return rc;
  if (int rc = tbh::make_tmap_2d(&tk, k, bf, 2, rows, (uint64_t)Hkv * D, (uint64_t)Hkv * D * 2, BLK, 64, 3)) return rc;
  if (int rc = tbh::make_tmap_2d(&tv, v, bf, 2, rows, (uint64_t)Hkv * D, (uint64_t)Hkv * D * 2, BLK, 64, 3)) return rc;
  FbParams p{};
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse; p.delta = delta; p.seq_start = seq_start;
  p.dK = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  p.dQ = dq32;
  p.status = status;
  const int smem = 6 * TILE + (int)sizeof(Ctl) + 1024;
  dim3 grid(S / BLK, Hkv, B);
  if (seq_start != nullptr) {
    TB_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    flash_bwd_kernel<true><<<grid, NTHREADS, smem, st>>>(tq, tdo, tk, tv, p);
  } else {
    TB_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    flash_bwd_kernel<false><<<grid, NTHREADS, smem, st>>>(tq, tdo, tk, tv, p);
  }
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
