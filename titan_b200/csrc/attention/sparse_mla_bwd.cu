// Sparse multi-head latent attention, backward: gradients of the queries and of the shared KV latent for the kernel
// of sparse_mla_fwd.cu, on tcgen05 tensor cores, memory O(S * top-k) (nothing of size [queries, keys] exists).
//
//   q [S, H, DQ], kv [T, DQ], idx [S, K] as in the forward;  dout [S, H, DV] bf16;  lse [S, H] fp32 (natural log,
//   sink included);  delta [S, H] fp32 = sum_d dout * out;
//   dq [S, H, DQ] bf16 (written),  dkv [T, DQ] fp32 (ACCUMULATED with vector reductions: zero it before the launch).
//
// One CTA works on one (query, head group) at a time and walks its selected keys in blocks of 128 gathered rows.
// With the tile Kt [128 keys x DQ] (its first DV columns are the values Vt), Q and dO of the head group [HG x .]:
//
//   S^T  [128 x HG] = Kt * Q^T              A = tile K-major,             B = Q  K-major
//   dP^T [128 x HG] = Vt * dO^T             A = tile K-major (DV cols),   B = dO K-major
//   P = exp(S * scale - lse),  dS = P * (dP - delta) * scale              (threads, one key per TMEM lane)
//   dQ^T [DQ x HG] += Kt^T * dS^T           A = tile MN-major,            B = dS [HG x 128 keys] K-major
//   dKV  [128 x DQ] = dS^T * Q  +  P^T * [dO | 0]
//                                           A = dS / P read MN-major (the same bytes that serve as B above),
//                                           B = Q / dO read MN-major
//
// dQ^T stays in tensor memory over all key blocks of the query.  dKV is produced per block in column groups of 192
// and added to the rows the block gathered from (different queries select the same rows): the group is staged as
// fp32 rows in the shared memory of the tile, which is dead by then, and every row leaves as ONE bulk reduction
// (`cp.reduce.async.bulk ... add.f32`, up to 768 contiguous bytes) instead of 48 vector atomics per thread.  When DQ is not a multiple of 128 the last 128-row block of dQ^T reads 64 columns past the tile; those
// accumulator lanes are never read.
//
// Every wait is bounded; a failure sets the status word and the CTA drains to the common exit.
//
// Replaces the reference's `npu_sparse_flash_attention_grad` / `sparse_flash_mla` backward
// (torchtitan_npu/converters/kernels/dsa.py:279-330, converters/kernels/npu_smla.py:422-660).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int BKEYS = 128;
constexpr int CHUNK_BYTES = 16384;   // [128 rows x 64 columns] bf16
constexpr int NTHREADS = 256;
constexpr int MAX_HG = 32;
constexpr int GROUP_COLS = 192;      // dKV columns per accumulator round (3 chunks of 64)
constexpr uint32_t TMEM_COLS = 512;  // S^T, dP^T (HG each), dQ^T (<= 5 * HG), dKV group (192)

struct BwdParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* kv;
  const int* idx;
  const __nv_bfloat16* dout;
  const float* lse;
  const float* delta;
  __nv_bfloat16* dq_out;
  float* dkv;
  int S, H, T, K;
  int dq, dv;
  float scale, scale_log2;
  int* status;
};

struct __align__(8) Ctl {
  uint64_t mma_bar;
  uint32_t tmem_slot;
  int abort_flag;
  float lse2[MAX_HG], delta[MAX_HG];
  int valid[BKEYS];
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld_row(uint32_t taddr, float* v, int n) {
  if (n == 16) {
    uint32_t r[16];
    tmem_ld_32x16(taddr, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
  } else {
    uint32_t r[32];
    tmem_ld_32x32(taddr, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
  }
}
__device__ __forceinline__ void st_shared_b16(uint32_t addr, float v) {
  const __nv_bfloat16 b = __float2bfloat16_rn(v);
  asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(*reinterpret_cast<const uint16_t*>(&b)) : "memory");
}

// fp32 staging of one dKV column group: [128 keys][w + 4] (the pad spreads the rows over the banks)
__host__ __device__ inline int stage_ld(int dq) { return (dq < GROUP_COLS ? dq : GROUP_COLS) + 4; }
__host__ __device__ inline int region0_bytes(int dq) {
  const int tile = (dq / 64) * CHUNK_BYTES, stage = BKEYS * stage_ld(dq) * 4;
  return ((tile > stage ? tile : stage) + 1023) & ~1023;
}

template <int HG>
__global__ void __launch_bounds__(NTHREADS, 1) sparse_mla_bwd_kernel(const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int qchunks = p.dq / 64, vchunks = p.dv / 64;
  constexpr int HROW = HG * 128;                 // bytes of one [HG x 64] chunk
  uint8_t* sK = smem;                            // qchunks x 16 KB: gathered tile [128 keys x dq]; later the dKV staging
  uint8_t* sQ = sK + region0_bytes(p.dq);        // qchunks x [HG x 64]
  uint8_t* sDO = sQ + qchunks * HROW;            // vchunks x [HG x 64]
  uint8_t* sP = sDO + vchunks * HROW;            // 2 x [HG x 64 keys]
  uint8_t* sDS = sP + 2 * HROW;                  // 2 x [HG x 64 keys]
  Ctl* ctl = reinterpret_cast<Ctl*>(sDS + 2 * HROW);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int groups = p.H / HG;
  const int nblocks = p.K / BKEYS;
  const int qb = (p.dq + 127) / 128;             // 128-row blocks of dQ^T
  const int ngroups = (p.dq + GROUP_COLS - 1) / GROUP_COLS;

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
  const uint32_t tmem_s = tmem;                  // S^T: HG columns
  const uint32_t tmem_dp = tmem + HG;            // dP^T: HG columns
  const uint32_t tmem_dq = tmem + 2 * HG;        // dQ^T: qb x HG columns
  const uint32_t tmem_kv = tmem + 2 * HG + 5 * HG;  // dKV group: up to 192 columns
  const uint32_t idesc_s = make_idesc_f16(128, HG, true, false, false);   // tile K-major, Q / dO K-major
  const uint32_t idesc_dq = make_idesc_f16(128, HG, true, true, false);   // tile MN-major, dS K-major
  uint32_t mma_phase = 0;
  volatile int* abort_flag = &ctl->abort_flag;
  const int r = ((warp & 3) << 5) | lane;        // TMEM lane of this thread (key row in S^T / dP^T / dKV)
  const uint32_t lane_off = ((uint32_t)((warp & 3) * 32)) << 16;
  const int half = warp >> 2;                    // the two warp sets split the columns of an epilogue

  for (long long item = blockIdx.x; item < (long long)p.S * groups && *abort_flag == 0; item += gridDim.x) {
    const int s = (int)(item / groups), g = (int)(item - (long long)s * groups);
    const long long hrow = (long long)s * p.H + (long long)g * HG;
    const __nv_bfloat16* qrow = p.q + hrow * p.dq;
    const __nv_bfloat16* dorow = p.dout + hrow * p.dv;
    const int* irow = p.idx + (long long)s * p.K;

    // ---- Q and dO of this (query, head group) as swizzled [HG x 64] chunks
    for (int i = tid; i < HG * qchunks * 8; i += NTHREADS) {
      const int h = i / (qchunks * 8), c = i - h * (qchunks * 8);
      const uint32_t dst = smem_u32(sQ) + (c >> 3) * HROW + h * 128 + (((c & 7) ^ (h & 7)) << 4);
      cp_async16(dst, qrow + (long long)h * p.dq + c * 8, 16);
    }
    for (int i = tid; i < HG * vchunks * 8; i += NTHREADS) {
      const int h = i / (vchunks * 8), c = i - h * (vchunks * 8);
      const uint32_t dst = smem_u32(sDO) + (c >> 3) * HROW + h * 128 + (((c & 7) ^ (h & 7)) << 4);
      cp_async16(dst, dorow + (long long)h * p.dv + c * 8, 16);
    }
    if (tid < HG) {
      ctl->lse2[tid] = p.lse[hrow + tid] * 1.4426950408889634f;
      ctl->delta[tid] = p.delta[hrow + tid];
    }

    for (int jb = 0; jb < nblocks; ++jb) {
      if (tid < BKEYS) {
        const int row = irow[jb * BKEYS + tid];
        ctl->valid[tid] = (row >= 0 && row < p.T) ? row : -1;
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the last group's rows have left the tile
      }
      __syncthreads();   // valid[] visible; the previous block's MMAs and epilogues have finished with smem / TMEM
      {
        // Thread = (row lane tid / 8, 16-byte piece tid % 8); it serves rows lane + 32 j of every chunk, so the row
        // pointers and the swizzled offset are computed once and each copy costs two additions.
        const int piece = tid & 7, rl = tid >> 3;
        const uint32_t dst0 = smem_u32(sK) + rl * 128 + ((piece ^ (rl & 7)) << 4);
        const __nv_bfloat16* src[BKEYS * 8 / NTHREADS];
        uint32_t nbytes[BKEYS * 8 / NTHREADS];
#pragma unroll
        for (int j = 0; j < BKEYS * 8 / NTHREADS; ++j) {
          const int row = ctl->valid[rl + j * (NTHREADS / 8)];
          src[j] = p.kv + (row >= 0 ? (long long)row * p.dq : 0ll) + piece * 8;
          nbytes[j] = row >= 0 ? 16u : 0u;         // an empty slot becomes a zero row
        }
        for (int ch = 0; ch < qchunks; ++ch) {
#pragma unroll
          for (int j = 0; j < BKEYS * 8 / NTHREADS; ++j)
            cp_async16(dst0 + ch * CHUNK_BYTES + j * (NTHREADS / 8) * 128, src[j] + ch * 64, nbytes[j]);
        }
      }
      cp_async_wait_all();
      fence_proxy_async();
      __syncthreads();

      // ---- S^T = Kt * Q^T and dP^T = Vt * dO^T
      if (tid == 0) {
        tc_fence_after();
        const uint32_t ka = smem_u32(sK), qa = smem_u32(sQ), da_ = smem_u32(sDO);
        for (int c = 0; c < qchunks; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = make_smem_desc(ka + c * CHUNK_BYTES + k * 32, 16, 1024, 2);
            const uint64_t db = make_smem_desc(qa + c * HROW + k * 32, 16, 1024, 2);
            umma_f16(tmem_s, da, db, idesc_s, (c > 0 || k > 0) ? 1u : 0u);
          }
        }
        for (int c = 0; c < vchunks; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = make_smem_desc(ka + c * CHUNK_BYTES + k * 32, 16, 1024, 2);
            const uint64_t db = make_smem_desc(da_ + c * HROW + k * 32, 16, 1024, 2);
            umma_f16(tmem_dp, da, db, idesc_s, (c > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(&ctl->mma_bar);
      }
      if (!mbar_wait(&ctl->mma_bar, mma_phase, abort_flag)) {
        if (tid == 0 && *abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_FULL); }
      }
      mma_phase ^= 1;
      tc_fence_after();
      __syncthreads();
      if (*abort_flag) break;

      // ---- P and dS (threads 0..127, one key each) into the two [HG x 128 keys] operand buffers
      if (tid < BKEYS) {
        float x[HG], dp[HG];
        tmem_ld_row(tmem_s + lane_off, x, HG);
        tmem_ld_row(tmem_dp + lane_off, dp, HG);
        tc_fence_before();
        const bool ok = ctl->valid[r] >= 0;
        const uint32_t off = (r >> 6) * HROW + ((r & 7) << 1);
        const int c16 = (r & 63) >> 3;
#pragma unroll
        for (int h = 0; h < HG; ++h) {
          const float pr = ok ? fast_exp2(x[h] * p.scale_log2 - ctl->lse2[h]) : 0.f;
          const float ds = pr * (dp[h] - ctl->delta[h]) * p.scale;
          const uint32_t a = off + h * 128 + ((c16 ^ (h & 7)) << 4);
          st_shared_b16(smem_u32(sP) + a, pr);
          st_shared_b16(smem_u32(sDS) + a, ds);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      __syncthreads();

      // ---- dQ^T += Kt^T * dS^T, then dKV in column groups
      for (int gi = 0; gi < ngroups; ++gi) {
        const int c0 = gi * GROUP_COLS;
        const int w = min(GROUP_COLS, p.dq - c0);              // columns of this group (multiple of 64)
        const int vw = max(0, min(w, p.dv - c0));              // of which the values' gradient also covers
        if (tid == 0) {
          tc_fence_after();
          const uint32_t ka = smem_u32(sK), pa = smem_u32(sP), dsa = smem_u32(sDS);
          if (gi == 0) {
            for (int mb = 0; mb < qb; ++mb) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {   // 16 keys per step: 16 rows x 128 B of the tile
                const uint64_t da = make_smem_desc(ka + (2 * mb) * CHUNK_BYTES + k * 2048, CHUNK_BYTES, 1024, 2);
                const uint64_t db = make_smem_desc(dsa + (k >> 2) * HROW + (k & 3) * 32, 16, 1024, 2);
                umma_f16(tmem_dq + mb * HG, da, db, idesc_dq, (jb > 0 || k > 0) ? 1u : 0u);
              }
            }
          }
          const uint32_t idesc_kv = make_idesc_f16(128, w, true, true, true);     // dS^T (MN-major) * Q (MN-major)
#pragma unroll
          for (int ks = 0; ks < HG / 16; ++ks) {   // 16 heads per step: 16 rows x 128 B
            const uint64_t da = make_smem_desc(dsa + ks * 2048, HROW, 1024, 2);
            const uint64_t db = make_smem_desc(smem_u32(sQ) + (c0 / 64) * HROW + ks * 2048, HROW, 1024, 2);
            umma_f16(tmem_kv, da, db, idesc_kv, ks > 0 ? 1u : 0u);
          }
          if (vw > 0) {
            const uint32_t idesc_v = make_idesc_f16(128, vw, true, true, true);   // P^T * dO
#pragma unroll
            for (int ks = 0; ks < HG / 16; ++ks) {
              const uint64_t da = make_smem_desc(pa + ks * 2048, HROW, 1024, 2);
              const uint64_t db = make_smem_desc(smem_u32(sDO) + (c0 / 64) * HROW + ks * 2048, HROW, 1024, 2);
              umma_f16(tmem_kv, da, db, idesc_v, 1u);
            }
          }
          umma_commit(&ctl->mma_bar);
        }
        // the previous group's row reductions drain from the staging area while these products run
        if (tid < BKEYS) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        if (!mbar_wait(&ctl->mma_bar, mma_phase, abort_flag)) {
          if (tid == 0 && *abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_FULL); }
        }
        mma_phase ^= 1;
        tc_fence_after();
        __syncthreads();
        if (*abort_flag) break;

        // ---- stage the group as fp32 rows (all 256 threads: two warp sets split the columns), then one bulk
        //      reduction per gathered row
        {
          const int row = ctl->valid[r];
          const int hw = w >> 1;                                 // columns per warp set (multiple of 32)
          const int ld = stage_ld(p.dq);
          const uint32_t srow = smem_u32(sK) + (uint32_t)(r * ld + half * hw) * 4;
          for (int c = 0; c < hw; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_kv + lane_off + half * hw + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + (uint32_t)(c + i) * 4), "r"(v[i]),
                           "r"(v[i + 1]), "r"(v[i + 2]), "r"(v[i + 3])
                           : "memory");
          }
          tc_fence_before();
          fence_proxy_async();   // the bulk engine reads what ordinary stores wrote
          __syncthreads();
          if (tid < BKEYS) {     // warps 0..3: r == tid
            if (row >= 0) {
              const float* dst = p.dkv + (long long)row * p.dq + c0;
              asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst),
                           "r"(smem_u32(sK) + (uint32_t)(r * ld) * 4), "r"(w * 4)
                           : "memory");
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            // the engine still reads the staging rows: whoever writes that region next (the next group's staging,
            // the next block's gather) is released by a barrier that follows this thread's wait_group.read
          }
        }
        __syncthreads();   // the group accumulator and the staging area are free again
      }
      if (*abort_flag) break;
    }
    if (*abort_flag) break;

    // ---- dQ^T (lane = column) -> dq[s, head, column]
    if (tid < BKEYS) {
      for (int mb = 0; mb < qb; ++mb) {
        const int col = mb * 128 + r;
        float o[HG];
        tmem_ld_row(tmem_dq + mb * HG + lane_off, o, HG);
        if (col < p.dq) {
#pragma unroll
          for (int h = 0; h < HG; ++h) p.dq_out[(hrow + h) * p.dq + col] = __float2bfloat16_rn(o[h]);
        }
      }
    }
    tc_fence_before();
    __syncthreads();
  }

  // The per-group waits above only cover the bulk engine's READS of the staging rows.  Before this CTA ends, wait for
  // the reductions themselves: a launch that completed while row updates were still on their way let the next
  // kernels of the stream read (and the allocator reuse) the gradient buffer too early.
  if (tid < BKEYS) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int HG>
int launch(const BwdParams& p, cudaStream_t st) {
  const int qchunks = p.dq / 64, vchunks = p.dv / 64;
  // the padded last dQ^T block (dq not a multiple of 128) reads one chunk past the tile: the Q / dO / P / dS buffers
  // that follow are at least that long for every accepted shape (dq >= 128 here; dq = 64 gets a spare chunk)
  const int spare = qchunks == 1 ? CHUNK_BYTES : 0;
  const int smem = region0_bytes(p.dq) + (qchunks + vchunks + 4) * HG * 128 + (int)sizeof(Ctl) + spare + 1024;
  TB_CUDA_CHECK(cudaFuncSetAttribute(sparse_mla_bwd_kernel<HG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long items = (long long)p.S * (p.H / HG);
  const int grid = (int)(items < sms ? items : sms);
  sparse_mla_bwd_kernel<HG><<<grid, NTHREADS, smem, st>>>(p);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
}  // namespace

// Shapes as in tb_sparse_mla_fwd.  `dkv` [T, dq] fp32 must be zero-filled by the caller (rows are accumulated);
// `dq_out` [S, H, dq] bf16 is overwritten.  `lse` is the forward's (natural log), `delta` = rowsum(dout * out).
TB_API int tb_sparse_mla_bwd(const void* q, const void* kv, const int* idx, const void* dout, const float* lse,
                             const float* delta, void* dq_out, float* dkv, int S, int H, int T, int K, int dq, int dv,
                             float scale, int* status, cudaStream_t st) {
  if (S <= 0) return 0;
  if (H < 16 || H % 16 || K < BKEYS || K % BKEYS || dq % 64 || dq > 576 || dv % 128 || dv > 512 || dv > dq || T < 1)
    return TB_ERR_ARG;
  BwdParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.kv = reinterpret_cast<const __nv_bfloat16*>(kv);
  p.idx = idx;
  p.dout = reinterpret_cast<const __nv_bfloat16*>(dout);
  p.lse = lse; p.delta = delta;
  p.dq_out = reinterpret_cast<__nv_bfloat16*>(dq_out);
  p.dkv = dkv;
  p.S = S; p.H = H; p.T = T; p.K = K; p.dq = dq; p.dv = dv;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  // 16 heads per CTA: with 32 the tile, Q, dO and the two operand buffers exceed the shared memory of an SM at dq 576
  return launch<16>(p, st);
}
