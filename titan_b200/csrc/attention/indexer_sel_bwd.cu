// Lightning-indexer backward at the SELECTED keys only, on tcgen05 tensor cores.
//
// The indexer scores every key, but its loss (KL against the attention's own distribution) only touches the top-k
// keys each query selected, so the gradient is sparse: for query s with selected key rows idx[s, j],
//
//   x[h, j]  = q[s, h, :] . k[idx_j, :]                    score[s, j] = sum_h w[s, h] * relu(x[h, j])
//   dx[h, j] = g[s, j] * w[s, h] * [x[h, j] > 0]
//   dq[s, h, :] = sum_j dx[h, j] * k[idx_j, :]             dw[s, h] = sum_j g[s, j] * relu(x[h, j])
//   dk[idx_j, :] += sum_h dx[h, j] * q[s, h, :]
//
// Work and traffic are O(S * top-k * H * D) instead of the O(S * T * H * D) of a dense backward over all T keys.
//
//   q [S, H, 128] bf16 (H = 16, 32 or 64 index heads), k [T, 128] bf16, idx [S, K] int32 (-1 = empty; K % 128 == 0),
//   g [S, K] fp32, w [S, H] fp32;  dq [S, H, 128] bf16, dw [S, H] fp32 (written), dk [T, 128] fp32 (ACCUMULATED).
//
// One CTA per query at a time, 128 gathered key rows per block (16-byte asynchronous copies into a 128-byte-swizzled
// tile; the next block's tile travels while this one is worked on):
//   X^T  [128 keys x H] = Kt * Q^T            A = tile K-major,   B = Q K-major
//   dX   -> bf16 [H x 128 keys] in shared memory (threads, one key per TMEM lane)
//   dQ^T [128 d x H]   += Kt^T * dX^T         A = tile MN-major,  B = dX K-major        (stays in tensor memory)
//   dK   [128 keys x 128 d] = dX^T * Q        A = dX MN-major,    B = Q MN-major
// and the dK rows leave as one 512-byte bulk reduction each (`cp.reduce.async.bulk ... add.f32`).
//
// Every wait is bounded; a failure sets the status word and the CTA drains to the common exit.
//
// Counterpart of the reference's lightning-indexer gradient inside its fused sparse-attention loss
// (torchtitan_npu/converters/kernels/dsa.py:332-420, models/deepseek_v32/model.py:363-420).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int D = 128;
constexpr int BKEYS = 128;
constexpr int BOX = 16384;           // [128 rows x 64 columns] bf16
constexpr int TILE = 2 * BOX;        // [128 keys x 128]
constexpr int NTHREADS = 256;
constexpr int MAX_H = 64;
constexpr int STAGE_LD = D + 4;      // fp32 staging rows of dK, padded against bank conflicts
constexpr uint32_t TMEM_COLS = 256;  // X^T (<= 64) | dQ^T (<= 64) | dK (128)

struct IsbParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const int* idx;
  const float* g;
  const float* w;
  __nv_bfloat16* dq;
  float* dw;
  float* dk;
  int S, H, T, K;
  int* status;
};

struct __align__(8) Ctl {
  uint64_t mma_bar;
  uint32_t tmem_slot;
  int abort_flag;
  float w[MAX_H];
  float red[4][MAX_H];
  int valid[2][BKEYS];
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int H>
__global__ void __launch_bounds__(NTHREADS, 1) indexer_sel_bwd_kernel(const IsbParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int HROW = H * 128;                  // bytes of one [H x 64] chunk
  uint8_t* sK = smem;                            // 2 tile buffers
  uint8_t* sQ = sK + 2 * TILE;                   // 2 chunks [H x 64 d]
  uint8_t* sDX = sQ + 2 * HROW;                  // 2 chunks [H x 64 keys]
  uint8_t* sStage = sDX + 2 * HROW;              // [128][STAGE_LD] fp32
  Ctl* ctl = reinterpret_cast<Ctl*>(sStage + BKEYS * STAGE_LD * 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nblocks = p.K / BKEYS;

  if (tid == 0) {
    mbar_init(&ctl->mma_bar, 1);
    ctl->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_slot;
  const uint32_t tmem_x = tmem, tmem_dq = tmem + 64, tmem_dk = tmem + 128;
  const uint32_t idesc_x = make_idesc_f16(128, H, true, false, false);    // tile K-major, Q K-major
  const uint32_t idesc_dq = make_idesc_f16(128, H, true, true, false);    // tile MN-major, dX K-major
  const uint32_t idesc_dk = make_idesc_f16(128, D, true, true, true);     // dX MN-major, Q MN-major
  uint32_t mma_phase = 0;
  volatile int* abort_flag = &ctl->abort_flag;
  const int r = ((warp & 3) << 5) | lane;        // TMEM lane of this thread
  const uint32_t lane_off = ((uint32_t)((warp & 3) * 32)) << 16;
  const int half = warp >> 2;

  for (int s = blockIdx.x; s < p.S && *abort_flag == 0; s += gridDim.x) {
    const __nv_bfloat16* qrow = p.q + (long long)s * H * D;
    const int* irow = p.idx + (long long)s * p.K;
    const float* grow = p.g + (long long)s * p.K;

    // gather of key block `blk` into tile buffer `buf` (all threads; asynchronous, one commit group per thread)
    auto gather = [&](int blk, int buf) {
      if (tid < BKEYS) {
        const int row = irow[blk * BKEYS + tid];
        ctl->valid[buf][tid] = (row >= 0 && row < p.T) ? row : -1;
      }
      const uint32_t base = smem_u32(sK) + buf * TILE;
      for (int i = tid; i < BKEYS * 16; i += NTHREADS) {
        const int kr = i >> 4, c = i & 15;
        int row = irow[blk * BKEYS + kr];
        if (row >= p.T) row = -1;
        const uint32_t dst = base + (c >> 3) * BOX + kr * 128 + (((c & 7) ^ (kr & 7)) << 4);
        const __nv_bfloat16* src = row >= 0 ? p.k + (long long)row * D + c * 8 : p.k;
        cp_async16(dst, src, row >= 0 ? 16 : 0);   // an empty slot becomes a zero row
      }
      cp_async_commit();
    };

    // Q of this query: H rows of 128 columns -> two swizzled [H x 64] chunks; the gate weights
    for (int i = tid; i < H * 16; i += NTHREADS) {
      const int h = i >> 4, c = i & 15;
      const uint32_t dst = smem_u32(sQ) + (c >> 3) * HROW + h * 128 + (((c & 7) ^ (h & 7)) << 4);
      cp_async16(dst, qrow + h * D + c * 8, 16);
    }
    if (tid < H) ctl->w[tid] = p.w[(long long)s * H + tid];
    gather(0, 0);

    float dwacc[H];                               // this lane's share of dw (threads 0..127)
#pragma unroll
    for (int h = 0; h < H; ++h) dwacc[h] = 0.f;

    for (int jb = 0; jb < nblocks; ++jb) {
      const int buf = jb & 1;
      const uint32_t tile = smem_u32(sK) + buf * TILE;
      cp_async_wait_all();
      fence_proxy_async();
      __syncthreads();   // the tile (and Q, w) is complete; the previous block is done with the other buffer
      if (jb + 1 < nblocks) gather(jb + 1, buf ^ 1);

      // ---- X^T = Kt * Q^T
      if (tid == 0) {
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_x, make_smem_desc(tile + c * BOX + k * 32, 16, 1024, 2),
                     make_smem_desc(qa + c * HROW + k * 32, 16, 1024, 2), idesc_x, (c | k) ? 1u : 0u);
        umma_commit(&ctl->mma_bar);
      }
      if (!mbar_wait(&ctl->mma_bar, mma_phase, abort_flag)) {
        if (tid == 0 && *abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_FULL); }
      }
      mma_phase ^= 1;
      tc_fence_after();
      __syncthreads();
      if (*abort_flag) break;

      // ---- dX (threads 0..127, one key each) -> bf16 [H x 128 keys]; dw partial sums
      if (tid < BKEYS) {
        const bool ok = ctl->valid[buf][r] >= 0;
        const float gj = ok ? grow[jb * BKEYS + r] : 0.f;
        const uint32_t off = (r >> 6) * HROW + ((r & 7) << 1);
        const int c16 = (r & 63) >> 3;
#pragma unroll
        for (int h0 = 0; h0 < H; h0 += 32) {
          constexpr int W = H < 32 ? H : 32;
          float x[W];
          if (W == 16) {
            uint32_t v[16];
            tmem_ld_32x16(tmem_x + lane_off + h0, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = __uint_as_float(v[i]);
          } else {
            uint32_t v[32];
            tmem_ld_32x32(tmem_x + lane_off + h0, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < W; ++i) x[i] = __uint_as_float(v[i]);
          }
#pragma unroll
          for (int i = 0; i < W; ++i) {
            const int h = h0 + i;
            const bool pos = x[i] > 0.f;
            const float dx = pos ? gj * ctl->w[h] : 0.f;
            dwacc[h] += pos ? gj * x[i] : 0.f;
            const __nv_bfloat16 b = __float2bfloat16_rn(dx);
            const uint32_t a = smem_u32(sDX) + off + h * 128 + ((c16 ^ (h & 7)) << 4);
            asm volatile("st.shared.b16 [%0], %1;" ::"r"(a), "h"(*reinterpret_cast<const uint16_t*>(&b)) : "memory");
          }
        }
        tc_fence_before();
      }
      fence_proxy_async();
      __syncthreads();

      // ---- dQ^T += Kt^T * dX^T ;  dK = dX^T * Q
      if (tid == 0) {
        tc_fence_after();
        const uint32_t xa = smem_u32(sDX), qa = smem_u32(sQ);
#pragma unroll
        for (int k = 0; k < 8; ++k)   // 16 keys per step: 16 rows x 128 B of the tile
          umma_f16(tmem_dq, make_smem_desc(tile + k * 2048, BOX, 1024, 2),
                   make_smem_desc(xa + (k >> 2) * HROW + (k & 3) * 32, 16, 1024, 2), idesc_dq,
                   (jb > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < H / 16; ++ks)   // 16 heads per step: 16 rows x 128 B
          umma_f16(tmem_dk, make_smem_desc(xa + ks * 2048, HROW, 1024, 2),
                   make_smem_desc(qa + ks * 2048, HROW, 1024, 2), idesc_dk, ks > 0 ? 1u : 0u);
        umma_commit(&ctl->mma_bar);
      }
      if (!mbar_wait(&ctl->mma_bar, mma_phase, abort_flag)) {
        if (tid == 0 && *abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_FULL); }
      }
      mma_phase ^= 1;
      tc_fence_after();
      __syncthreads();
      if (*abort_flag) break;

      // ---- dK rows: tensor memory -> fp32 staging rows (all 256 threads) -> one bulk reduction per gathered row
      {
        const uint32_t srow = smem_u32(sStage) + (uint32_t)(r * STAGE_LD + half * 64) * 4;
#pragma unroll 1
        for (int c = 0; c < 64; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_dk + lane_off + half * 64 + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + (uint32_t)(c + i) * 4), "r"(v[i]),
                         "r"(v[i + 1]), "r"(v[i + 2]), "r"(v[i + 3])
                         : "memory");
        }
        tc_fence_before();
        fence_proxy_async();
        __syncthreads();
        if (tid < BKEYS) {
          const int row = ctl->valid[buf][r];
          if (row >= 0)
            asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(
                             p.dk + (long long)row * D),
                         "r"(smem_u32(sStage) + (uint32_t)(r * STAGE_LD) * 4), "r"(D * 4)
                         : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        }
      }
      // no barrier needed here: the next iteration starts with one, and nothing before it touches the staging rows
    }
    if (*abort_flag) break;

    // ---- dQ^T (lane = column d) -> dq[s, h, d]; dw: lanes of a warp, then the four warps
    if (tid < BKEYS) {
#pragma unroll
      for (int h0 = 0; h0 < H; h0 += 32) {
        constexpr int W = H < 32 ? H : 32;
        if (W == 16) {
          uint32_t v[16];
          tmem_ld_32x16(tmem_dq + lane_off + h0, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            p.dq[((long long)s * H + h0 + i) * D + r] = __float2bfloat16_rn(__uint_as_float(v[i]));
        } else {
          uint32_t v[32];
          tmem_ld_32x32(tmem_dq + lane_off + h0, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < W; ++i)
            p.dq[((long long)s * H + h0 + i) * D + r] = __float2bfloat16_rn(__uint_as_float(v[i]));
        }
      }
      tc_fence_before();
#pragma unroll
      for (int h = 0; h < H; ++h) {
        const float v = warp_sum(dwacc[h]);
        if (lane == 0) ctl->red[warp][h] = v;
      }
    }
    __syncthreads();
    if (tid < H)
      p.dw[(long long)s * H + tid] = ctl->red[0][tid] + ctl->red[1][tid] + ctl->red[2][tid] + ctl->red[3][tid];
    __syncthreads();   // tensor memory, Q and the control block are free for the next query
  }

  cp_async_wait_all();
  if (tid < BKEYS) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the reductions themselves, not only their reads
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int H>
int launch(const IsbParams& p, cudaStream_t st) {
  const int smem = 2 * TILE + 4 * H * 128 + BKEYS * STAGE_LD * 4 + (int)sizeof(Ctl) + 1024;
  TB_CUDA_CHECK(cudaFuncSetAttribute(indexer_sel_bwd_kernel<H>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = p.S < sms ? p.S : sms;
  indexer_sel_bwd_kernel<H><<<grid, NTHREADS, smem, st>>>(p);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
}  // namespace

// q [S, H, 128] bf16, k [T, 128] bf16, idx [S, K] int32 (-1 = empty slot, K a multiple of 128), g [S, K] fp32 (the
// gradient of the score at each selected key), w [S, H] fp32 → dq [S, H, 128] bf16, dw [S, H] fp32 (both written),
// dk [T, 128] fp32 (rows accumulated: zero it before the launch).  H is 16, 32 or 64.
TB_API int tb_indexer_sel_bwd(const void* q, const void* k, const int* idx, const float* g, const float* w, void* dq,
                              float* dw, float* dk, int S, int H, int T, int K, int head_dim, int* status,
                              cudaStream_t st) {
  if (S <= 0) return 0;
  if (head_dim != D || K < BKEYS || K % BKEYS || T < 1 || (H != 16 && H != 32 && H != 64)) return TB_ERR_ARG;
  IsbParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.k = reinterpret_cast<const __nv_bfloat16*>(k);
  p.idx = idx; p.g = g; p.w = w;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  p.dw = dw; p.dk = dk;
  p.S = S; p.H = H; p.T = T; p.K = K;
  p.status = status;
  if (H == 64) return launch<64>(p, st);
  if (H == 32) return launch<32>(p, st);
  return launch<16>(p, st);
}
