// Sparse multi-head latent attention, forward: every query attends ONLY to its selected keys of the shared one-head
// KV latent (DeepSeek sparse attention / MLA absorb layout), on tcgen05 tensor cores, memory O(S * top-k).
//
//   q    [S, H, DQ]  bf16   queries of all heads (DQ = kv_lora + rope dims, e.g. 576)
//   kv   [T, DQ]     bf16   shared latent keys; the VALUES are the first DV columns of the same rows (e.g. 512)
//   idx  [S, K]      int32  selected key rows per query, -1 = empty slot; K a multiple of 128
//   out  [S, H, DV]  bf16,  lse [S, H] fp32 (natural log),  teacher [S, K] fp32 = sum over heads of the softmax
//   sink [H] fp32 or null   a per-head logit that joins the softmax denominator only (sink attention)
//
// One CTA works on one (query, head group) at a time.  The selected rows of a 128-key block are GATHERED into shared
// memory with 16-byte asynchronous copies into the 128-byte-swizzled tile layout (empty slots are zero-filled), and
// the same tile feeds both contractions:
//
//   S^T [128 keys x HG heads] = K_tile [128 x DQ]  * Q^T      A = the tile read K-major,  B = Q K-major
//   O^T [DV x HG]            += V_tile^T [DV x 128] * P^T     A = the SAME tile read MN-major (rows = contraction),
//                                                              B = P [HG x 128 keys] K-major, written by the softmax
//
// Keys sit on the M axis (TMEM lane = key), heads on the N axis, so the few heads of a latent-attention model
// (16 .. 32 per group) cost N = 16 .. 32 columns instead of padding M to 128.  The softmax runs along the lanes:
// per-head maxima and sums are reduced with warp shuffles and a small shared-memory exchange.
//
// Two passes over the key blocks: the first finds the exact row maxima and sums, the second computes the
// probabilities against them, so the head-summed probabilities (the indexer's teacher) are exact and O^T never needs
// rescaling.  When the logits of all blocks fit in tensor memory next to O^T (K / 128 + DV / 128 blocks of HG columns
// <= 512 columns: top-2048 with 16 heads does) the first pass leaves them there, and the second pass only gathers the
// value columns again: its softmax runs on the stashed logits WHILE the copies are in flight and no logit is computed
// twice.  Otherwise the second pass repeats gather and logits.
//
// Every wait is bounded; a failure sets the status word and the CTA drains to the common exit.
//
// Replaces the reference's `npu_sparse_flash_attention` / `sparse_flash_mla` forward
// (torchtitan_npu/converters/kernels/dsa.py:195-277, converters/kernels/npu_smla.py:59-420).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int BKEYS = 128;          // keys per block = M of both MMAs
constexpr int CHUNK_BYTES = 16384;  // one [128 rows x 64 columns] bf16 chunk of the gathered tile
constexpr int NTHREADS = 256;
constexpr int MAX_HG = 32;          // heads per CTA
constexpr uint32_t TMEM_COLS = 512; // O^T (DV/128 * HG) + S^T (HG, or K/128 * HG when the logits are stashed)

struct SmlaParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* kv;
  const int* idx;
  __nv_bfloat16* out;
  float* lse;
  float* teacher;
  const float* sink;
  int S, H, T, K;
  int dq, dv;          // multiples of 64 / 128
  int hg;              // heads per CTA (16 or 32), H % hg == 0
  float scale_log2;    // softmax scale * log2(e)
  int teacher_atomic;  // several head groups add into teacher
  int stash;           // the logits of all key blocks stay in tensor memory between the passes
  int pipelined;       // half-tile ring (needs `stash`)
  int* status;
};

struct __align__(8) Ctl {
  uint64_t mma_bar;
  uint32_t tmem_slot;
  int abort_flag;
  float m[MAX_HG], l[MAX_HG], inv_l[MAX_HG];
  float red[4][MAX_HG];
  int valid[2][BKEYS];   // row ids of the current and of the next key block
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {   // arguments are <= 0 here; -inf gives 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld_row(uint32_t taddr, float* v, int n) {  // n = 16 or 32 columns
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

template <int HG>
__global__ void __launch_bounds__(NTHREADS, 1) sparse_mla_fwd_kernel(const SmlaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int qchunks = p.dq / 64;                 // 64-column chunks of a key row / a query row
  uint8_t* sK = smem;                            // qchunks x 16 KB: gathered tile [128 keys x dq]
  uint8_t* sQ = sK + qchunks * CHUNK_BYTES;      // qchunks x (HG x 128 B): Q of this head group
  uint8_t* sP = sQ + qchunks * HG * 128;         // 2 x (HG x 128 B): P [HG x 128 keys]
  Ctl* ctl = reinterpret_cast<Ctl*>(sP + 2 * HG * 128);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int groups = p.H / HG;
  const int nblocks = p.K / BKEYS;
  const int dvb = p.dv / 128;                    // 128-row blocks of O^T

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
  const uint32_t tmem_o = tmem;                  // O^T: dvb x HG columns
  const uint32_t tmem_s0 = tmem + dvb * HG;      // S^T: HG columns per key block (one block unless stashed)
  const int vchunks = p.dv / 64;
  const uint32_t idesc_s = make_idesc_f16(128, HG, true, false, false);   // K tile K-major, Q K-major
  const uint32_t idesc_o = make_idesc_f16(128, HG, true, true, false);    // V tile MN-major, P K-major
  uint32_t mma_phase = 0;
  volatile int* abort_flag = &ctl->abort_flag;
  const int r = tid;                             // softmax threads: tid < 128, TMEM lane = key row r
  const uint32_t lane_off = ((uint32_t)((warp & 3) * 32)) << 16;

  for (long long item = blockIdx.x; item < (long long)p.S * groups && *abort_flag == 0; item += gridDim.x) {
    const int s = (int)(item / groups), g = (int)(item - (long long)s * groups);
    const __nv_bfloat16* qrow = p.q + ((long long)s * p.H + (long long)g * HG) * p.dq;
    const int* irow = p.idx + (long long)s * p.K;

    // ---- Q of this (query, head group): HG rows of dq columns -> qchunks swizzled [HG x 64] chunks
    for (int i = tid; i < HG * qchunks * 8; i += NTHREADS) {
      const int h = i / (qchunks * 8), c = i - h * (qchunks * 8);
      const uint32_t dst = smem_u32(sQ) + (c >> 3) * (HG * 128) + h * 128 + (((c & 7) ^ (h & 7)) << 4);
      cp_async16(dst, qrow + (long long)h * p.dq + c * 8, 16);
    }
    if (tid < HG) {
      const float sk = p.sink != nullptr ? p.sink[g * HG + tid] * 1.4426950408889634f : -INFINITY;
      ctl->m[tid] = sk;                          // the sink joins the maximum and the denominator
      ctl->l[tid] = p.sink != nullptr ? 1.f : 0.f;
    }

    // Steps t = pass * nblocks + jb.  The gather of step t + 1 is issued as soon as step t no longer needs the tile
    // (after its logits in the first pass, after its value product in the second), so the copies travel under the
    // softmax work; row ids alternate between two small buffers.
    auto issue_gather = [&](int t) {
      const int tpass = t >= nblocks ? 1 : 0, tjb = t - tpass * nblocks;
      const int nch = (tpass == 1 && p.stash) ? vchunks : qchunks;   // stashed logits: only the value columns
      int* valid = ctl->valid[t & 1];
      if (tid < BKEYS) {
        const int row = irow[tjb * BKEYS + tid];
        valid[tid] = (row >= 0 && row < p.T) ? row : -1;
      }
      __syncthreads();   // row ids first (one global read each), then the copies look them up in shared memory
      // Thread = (row lane tid / 8, 16-byte piece tid % 8); it serves rows lane + 32 j of every chunk, so the row
      // pointers and the swizzled offset are computed once and each copy costs two additions.
      const int piece = tid & 7, rl = tid >> 3;
      const uint32_t dst0 = smem_u32(sK) + rl * 128 + ((piece ^ (rl & 7)) << 4);
      const __nv_bfloat16* src[BKEYS * 8 / NTHREADS];
      uint32_t nbytes[BKEYS * 8 / NTHREADS];
#pragma unroll
      for (int j = 0; j < BKEYS * 8 / NTHREADS; ++j) {
        const int row = valid[rl + j * (NTHREADS / 8)];
        src[j] = p.kv + (row >= 0 ? (long long)row * p.dq : 0ll) + piece * 8;
        nbytes[j] = row >= 0 ? 16u : 0u;           // an empty slot becomes a zero row
      }
      for (int ch = 0; ch < nch; ++ch) {
#pragma unroll
        for (int j = 0; j < BKEYS * 8 / NTHREADS; ++j)
          cp_async16(dst0 + ch * CHUNK_BYTES + j * (NTHREADS / 8) * 128, src[j] + ch * 64, nbytes[j]);
      }
    };
    issue_gather(0);

    for (int pass = 0; pass < 2; ++pass) {
      for (int jb = 0; jb < nblocks; ++jb) {
        const int t = pass * nblocks + jb;
        const bool reuse = pass == 1 && p.stash;     // logits of this block are in tensor memory already
        const uint32_t tmem_s = tmem_s0 + (p.stash ? jb * HG : 0);
        const int* valid = ctl->valid[t & 1];
        if (!reuse) {
          cp_async_wait_all();
          fence_proxy_async();   // generic-proxy writes -> visible to the tensor cores (async proxy)
          __syncthreads();

          // ---- S^T = K_tile * Q^T
          if (tid == 0) {
            tc_fence_after();
            const uint32_t ka = smem_u32(sK), qa = smem_u32(sQ);
            for (int c = 0; c < qchunks; ++c) {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint64_t da = make_smem_desc(ka + c * CHUNK_BYTES + k * 32, 16, 1024, 2);
                const uint64_t db = make_smem_desc(qa + c * (HG * 128) + k * 32, 16, 1024, 2);
                umma_f16(tmem_s, da, db, idesc_s, (c > 0 || k > 0) ? 1u : 0u);
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
          if (pass == 0) issue_gather(t + 1);   // the tile is free: the next block (or the second pass) travels now
        }

        // ---- softmax along the lanes (threads 0..127, one key each)
        float x[HG];
        if (tid < BKEYS) {
          tmem_ld_row(tmem_s + lane_off, x, HG);
          const bool ok = valid[r] >= 0;
#pragma unroll
          for (int h = 0; h < HG; ++h) x[h] = ok ? x[h] * p.scale_log2 : -INFINITY;
          tc_fence_before();   // the next MMA into S^T is ordered after these reads
        }
        if (pass == 0) {
          // block maxima per head, then the running (max, sum) update
          if (tid < BKEYS) {
#pragma unroll
            for (int h = 0; h < HG; ++h) {
              const float v = warp_max(x[h]);
              if (lane == 0) ctl->red[warp][h] = v;
            }
          }
          __syncthreads();
          float m_new = 0.f;
          if (tid < HG) {
            const float bm = fmaxf(fmaxf(ctl->red[0][tid], ctl->red[1][tid]), fmaxf(ctl->red[2][tid], ctl->red[3][tid]));
            const float m_old = ctl->m[tid];
            m_new = fmaxf(m_old, bm);
            ctl->l[tid] = (m_new == -INFINITY) ? 0.f : ctl->l[tid] * exp2f(m_old - m_new);
            ctl->m[tid] = m_new;
          }
          __syncthreads();
          if (tid < BKEYS) {
#pragma unroll
            for (int h = 0; h < HG; ++h) {
              const float mh = ctl->m[h];
              const float e = (x[h] == -INFINITY) ? 0.f : fast_exp2(x[h] - mh);
              const float v = warp_sum(e);
              if (lane == 0) ctl->red[warp][h] = v;
            }
          }
          __syncthreads();
          if (tid < HG) ctl->l[tid] += ctl->red[0][tid] + ctl->red[1][tid] + ctl->red[2][tid] + ctl->red[3][tid];
          __syncthreads();
        } else {
          // exact probabilities: teacher and the P operand; then O^T += V^T * P^T
          if (tid < BKEYS) {
            float t = 0.f;
            const uint32_t pbase = smem_u32(sP) + (r >> 6) * (HG * 128) + ((r & 7) << 1);
            const int c16 = (r & 63) >> 3;
#pragma unroll
            for (int h = 0; h < HG; ++h) {
              const float e = (x[h] == -INFINITY) ? 0.f : fast_exp2(x[h] - ctl->m[h]);
              t += e * ctl->inv_l[h];
              const __nv_bfloat16 b = __float2bfloat16_rn(e);
              const uint32_t addr = pbase + h * 128 + ((c16 ^ (h & 7)) << 4);
              asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(*reinterpret_cast<const uint16_t*>(&b)) : "memory");
            }
            if (p.teacher != nullptr) {
              float* dst = p.teacher + (long long)s * p.K + jb * BKEYS + r;
              if (p.teacher_atomic) atomicAdd(dst, t); else *dst = t;
            }
          }
          cp_async_wait_all();   // with stashed logits the value tile was travelling during the softmax above
          fence_proxy_async();
          tc_fence_before();
          __syncthreads();
          if (tid == 0) {
            tc_fence_after();
            const uint32_t ka = smem_u32(sK), pa = smem_u32(sP);
            for (int mb = 0; mb < dvb; ++mb) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {   // 16 keys per step: 16 rows x 128 B of the tile
                const uint64_t da = make_smem_desc(ka + (2 * mb) * CHUNK_BYTES + k * 2048, CHUNK_BYTES, 1024, 2);
                const uint64_t db = make_smem_desc(pa + (k >> 2) * (HG * 128) + (k & 3) * 32, 16, 1024, 2);
                umma_f16(tmem_o + mb * HG, da, db, idesc_o, (jb > 0 || k > 0) ? 1u : 0u);
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
          if (t + 1 < 2 * nblocks) issue_gather(t + 1);   // the tile is free again
        }
      }
      if (*abort_flag) break;
      if (pass == 0) {
        if (tid < HG) {
          const float l = ctl->l[tid];
          ctl->inv_l[tid] = l > 0.f ? 1.f / l : 0.f;
          if (p.lse != nullptr)
            p.lse[(long long)s * p.H + g * HG + tid] =
                l > 0.f ? (ctl->m[tid] + log2f(l)) * 0.6931471805599453f : -INFINITY;
        }
        __syncthreads();
      }
    }
    if (*abort_flag) break;

    // ---- O^T (lane = value column) -> out[s, head, column], normalised
    if (tid < BKEYS) {
      for (int mb = 0; mb < dvb; ++mb) {
        float o[HG];
        tmem_ld_row(tmem_o + mb * HG + lane_off, o, HG);
        tc_fence_before();
#pragma unroll
        for (int h = 0; h < HG; ++h)
          p.out[((long long)s * p.H + g * HG + h) * p.dv + mb * 128 + r] = __float2bfloat16_rn(o[h] * ctl->inv_l[h]);
      }
    }
    tc_fence_before();
    __syncthreads();   // TMEM and the control block are free for the next item
  }

  cp_async_wait_all();   // a CTA that gave up may still have copies in flight
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Pipelined form for the stashed-logit case: the tile is split into two half-tiles of chunks that alternate between
// two buffers, so the copies of one half travel while the tensor cores work on the other and while the softmax
// threads handle the block.  Half-steps u = ((pass * nblocks + jb) * 2 + half); every thread commits exactly one
// copy group per half-step and waits with one group left in flight.
//   pass 0, half h: logits of block jb accumulate over the half's chunks (first the lower, then the upper columns)
//   pass 1, half h: the value product of O^T row blocks that live in this half's chunk pairs
template <int HG>
__global__ void __launch_bounds__(NTHREADS, 1) sparse_mla_fwd_pipe_kernel(const SmlaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int qchunks = p.dq / 64, vchunks = p.dv / 64;
  const int hchunks = (qchunks + 1) / 2;         // chunks a half buffer holds
  const int half_bytes = hchunks * CHUNK_BYTES;
  uint8_t* sK = smem;                            // 2 half buffers
  uint8_t* sQ = sK + 2 * half_bytes;
  uint8_t* sP = sQ + qchunks * HG * 128;
  Ctl* ctl = reinterpret_cast<Ctl*>(sP + 2 * HG * 128);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int groups = p.H / HG;
  const int nblocks = p.K / BKEYS;
  const int dvb = p.dv / 128;

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
  const uint32_t tmem_o = tmem;
  const uint32_t tmem_s0 = tmem + dvb * HG;      // stashed logits: HG columns per key block
  const uint32_t idesc_s = make_idesc_f16(128, HG, true, false, false);
  const uint32_t idesc_o = make_idesc_f16(128, HG, true, true, false);
  uint32_t mma_phase = 0;
  volatile int* abort_flag = &ctl->abort_flag;
  const int r = tid;
  const uint32_t lane_off = ((uint32_t)((warp & 3) * 32)) << 16;
  const int U = 4 * nblocks;                     // half-steps per item

  for (long long item = blockIdx.x; item < (long long)p.S * groups && *abort_flag == 0; item += gridDim.x) {
    const int s = (int)(item / groups), g = (int)(item - (long long)s * groups);
    const __nv_bfloat16* qrow = p.q + ((long long)s * p.H + (long long)g * HG) * p.dq;
    const int* irow = p.idx + (long long)s * p.K;

    for (int i = tid; i < HG * qchunks * 8; i += NTHREADS) {
      const int h = i / (qchunks * 8), c = i - h * (qchunks * 8);
      const uint32_t dst = smem_u32(sQ) + (c >> 3) * (HG * 128) + h * 128 + (((c & 7) ^ (h & 7)) << 4);
      cp_async16(dst, qrow + (long long)h * p.dq + c * 8, 16);
    }
    if (tid < HG) {
      const float sk = p.sink != nullptr ? p.sink[g * HG + tid] * 1.4426950408889634f : -INFINITY;
      ctl->m[tid] = sk;
      ctl->l[tid] = p.sink != nullptr ? 1.f : 0.f;
    }

    // chunk range of half-step u, its block and pass
    auto decode = [&](int u, int& pass, int& jb, int& half, int& c0, int& c1) {
      pass = u >= 2 * nblocks ? 1 : 0;
      const int rem = u - pass * 2 * nblocks;
      jb = rem >> 1; half = rem & 1;
      const int split = pass == 0 ? hchunks : vchunks / 2, end = pass == 0 ? qchunks : vchunks;
      c0 = half ? split : 0;
      c1 = half ? end : split;
    };
    auto issue = [&](int u) {
      int pass, jb, half, c0, c1;
      decode(u, pass, jb, half, c0, c1);
      int* valid = ctl->valid[(pass * nblocks + jb) & 1];
      if (half == 0) {                           // row ids of the block, once
        if (tid < BKEYS) {
          const int row = irow[jb * BKEYS + tid];
          valid[tid] = (row >= 0 && row < p.T) ? row : -1;
        }
        __syncthreads();
      }
      const uint32_t base = smem_u32(sK) + (u & 1) * half_bytes;
      const int piece = tid & 7, rl = tid >> 3;   // thread = (row lane, 16-byte piece): rows rl + 32 j of every chunk
      const uint32_t dst0 = base + rl * 128 + ((piece ^ (rl & 7)) << 4);
      const __nv_bfloat16* src[BKEYS * 8 / NTHREADS];
      uint32_t nbytes[BKEYS * 8 / NTHREADS];
#pragma unroll
      for (int j = 0; j < BKEYS * 8 / NTHREADS; ++j) {
        const int row = valid[rl + j * (NTHREADS / 8)];
        src[j] = p.kv + (row >= 0 ? (long long)row * p.dq : 0ll) + c0 * 64 + piece * 8;
        nbytes[j] = row >= 0 ? 16u : 0u;
      }
      for (int ch = 0; ch < c1 - c0; ++ch) {
#pragma unroll
        for (int j = 0; j < BKEYS * 8 / NTHREADS; ++j)
          cp_async16(dst0 + ch * CHUNK_BYTES + j * (NTHREADS / 8) * 128, src[j] + ch * 64, nbytes[j]);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue(0);
    issue(1);

    for (int u = 0; u < U; ++u) {
      int pass, jb, half, c0, c1;
      decode(u, pass, jb, half, c0, c1);
      const uint32_t tmem_s = tmem_s0 + jb * HG;
      const int* valid = ctl->valid[(pass * nblocks + jb) & 1];
      const uint32_t base = smem_u32(sK) + (u & 1) * half_bytes;

      if (pass == 1 && half == 0 && tid < BKEYS) {
        // exact probabilities of block jb from the stashed logits, while this block's value copies travel
        float x[HG];
        tmem_ld_row(tmem_s + lane_off, x, HG);
        const bool ok = valid[r] >= 0;
        float t = 0.f;
        const uint32_t pbase = smem_u32(sP) + (r >> 6) * (HG * 128) + ((r & 7) << 1);
        const int c16 = (r & 63) >> 3;
#pragma unroll
        for (int h = 0; h < HG; ++h) {
          const float e = ok ? exp2f(x[h] * p.scale_log2 - ctl->m[h]) : 0.f;
          t += e * ctl->inv_l[h];
          const __nv_bfloat16 b = __float2bfloat16_rn(e);
          const uint32_t addr = pbase + h * 128 + ((c16 ^ (h & 7)) << 4);
          asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(*reinterpret_cast<const uint16_t*>(&b)) : "memory");
        }
        if (p.teacher != nullptr) {
          float* dst = p.teacher + (long long)s * p.K + jb * BKEYS + r;
          if (p.teacher_atomic) atomicAdd(dst, t); else *dst = t;
        }
        tc_fence_before();
      }
      if (u + 1 < U) asm volatile("cp.async.wait_group 1;" ::: "memory");
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      fence_proxy_async();
      __syncthreads();

      if (tid == 0) {
        tc_fence_after();
        if (pass == 0) {
          const uint32_t qa = smem_u32(sQ);
          for (int c = c0; c < c1; ++c) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint64_t da = make_smem_desc(base + (c - c0) * CHUNK_BYTES + k * 32, 16, 1024, 2);
              const uint64_t db = make_smem_desc(qa + c * (HG * 128) + k * 32, 16, 1024, 2);
              umma_f16(tmem_s, da, db, idesc_s, (half > 0 || c > c0 || k > 0) ? 1u : 0u);
            }
          }
        } else {
          const uint32_t pa = smem_u32(sP);
          for (int mb = c0 / 2; mb < c1 / 2; ++mb) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint64_t da = make_smem_desc(base + (2 * mb - c0) * CHUNK_BYTES + k * 2048, CHUNK_BYTES, 1024, 2);
              const uint64_t db = make_smem_desc(pa + (k >> 2) * (HG * 128) + (k & 3) * 32, 16, 1024, 2);
              umma_f16(tmem_o + mb * HG, da, db, idesc_o, (jb > 0 || k > 0) ? 1u : 0u);
            }
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
      if (u + 2 < U) issue(u + 2);               // this half buffer is free: the half after next travels now

      if (pass == 0 && half == 1) {
        // running (max, sum) of block jb while the next block's copies travel
        float x[HG];
        if (tid < BKEYS) {
          tmem_ld_row(tmem_s + lane_off, x, HG);
          const bool ok = valid[r] >= 0;
#pragma unroll
          for (int h = 0; h < HG; ++h) {
            x[h] = ok ? x[h] * p.scale_log2 : -INFINITY;
            const float v = warp_max(x[h]);
            if (lane == 0) ctl->red[warp][h] = v;
          }
          tc_fence_before();
        }
        __syncthreads();
        if (tid < HG) {
          const float bm = fmaxf(fmaxf(ctl->red[0][tid], ctl->red[1][tid]), fmaxf(ctl->red[2][tid], ctl->red[3][tid]));
          const float m_old = ctl->m[tid];
          const float m_new = fmaxf(m_old, bm);
          ctl->l[tid] = (m_new == -INFINITY) ? 0.f : ctl->l[tid] * exp2f(m_old - m_new);
          ctl->m[tid] = m_new;
        }
        __syncthreads();
        if (tid < BKEYS) {
#pragma unroll
          for (int h = 0; h < HG; ++h) {
            const float e = (x[h] == -INFINITY) ? 0.f : fast_exp2(x[h] - ctl->m[h]);
            const float v = warp_sum(e);
            if (lane == 0) ctl->red[warp][h] = v;
          }
        }
        __syncthreads();
        if (tid < HG) ctl->l[tid] += ctl->red[0][tid] + ctl->red[1][tid] + ctl->red[2][tid] + ctl->red[3][tid];
        if (jb == nblocks - 1 && tid < HG) {      // end of the first pass: normalisers and the log-sum-exp
          const float l = ctl->l[tid];
          ctl->inv_l[tid] = l > 0.f ? 1.f / l : 0.f;
          if (p.lse != nullptr)
            p.lse[(long long)s * p.H + g * HG + tid] =
                l > 0.f ? (ctl->m[tid] + log2f(l)) * 0.6931471805599453f : -INFINITY;
        }
        __syncthreads();
      }
    }
    if (*abort_flag) break;

    if (tid < BKEYS) {
      for (int mb = 0; mb < dvb; ++mb) {
        float o[HG];
        tmem_ld_row(tmem_o + mb * HG + lane_off, o, HG);
        tc_fence_before();
#pragma unroll
        for (int h = 0; h < HG; ++h)
          p.out[((long long)s * p.H + g * HG + h) * p.dv + mb * 128 + r] = __float2bfloat16_rn(o[h] * ctl->inv_l[h]);
      }
    }
    tc_fence_before();
    __syncthreads();
  }

  asm volatile("cp.async.wait_group 0;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int HG>
int launch(const SmlaParams& p, cudaStream_t st) {
  const int qchunks = p.dq / 64, vchunks = p.dv / 64;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long items = (long long)p.S * (p.H / HG);
  const int grid = (int)(items < sms ? items : sms);
  const int tail = qchunks * HG * 128 + 2 * HG * 128 + (int)sizeof(Ctl) + 1024;
  // stashed logits and value chunks that split into two halves of whole chunk pairs: the pipelined form
  const int hchunks = (qchunks + 1) / 2;
  const int smem_pipe = 2 * hchunks * CHUNK_BYTES + tail;
  if (p.stash && p.pipelined && vchunks % 4 == 0 && vchunks / 2 <= hchunks && smem_pipe <= 227 * 1024) {
    TB_CUDA_CHECK(cudaFuncSetAttribute(sparse_mla_fwd_pipe_kernel<HG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       smem_pipe));
    sparse_mla_fwd_pipe_kernel<HG><<<grid, NTHREADS, smem_pipe, st>>>(p);
  } else {
    const int smem = qchunks * CHUNK_BYTES + tail;
    TB_CUDA_CHECK(cudaFuncSetAttribute(sparse_mla_fwd_kernel<HG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    sparse_mla_fwd_kernel<HG><<<grid, NTHREADS, smem, st>>>(p);
  }
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
}  // namespace

// q [S, H, dq], kv [T, dq] (values = first dv columns), idx [S, K] int32 (-1 = empty), out [S, H, dv],
// lse [S, H] (may be null), teacher [S, K] (may be null; must be zero-filled when H > 32), sink [H] (may be null).
// Requirements: bf16; dq a multiple of 64 up to 576; dv a multiple of 128 up to 512 and <= dq; K a multiple of 128;
// H a multiple of 16.
static int g_sparse_mla_pipelined = 0;

// 0 (default): the single-tile kernel; 1: the half-tile ring where it applies.  Measured at 4096 queries x 16 heads x
// top-2048: 7.1 ms single tile, 7.7 ms ring: the block is bound by its chain of dependent steps (row ids, copies,
// fence, product, commit, wait, softmax), not by the copies the ring hides, and the ring doubles the number of
// product / wait round trips.  Kept as an option and tested against the single-tile kernel.
TB_API int tb_sparse_mla_fwd_set_pipelined(int on) {
  g_sparse_mla_pipelined = on ? 1 : 0;
  return 0;
}

TB_API int tb_sparse_mla_fwd(const void* q, const void* kv, const int* idx, void* out, float* lse, float* teacher,
                             const float* sink, int S, int H, int T, int K, int dq, int dv, float scale, int* status,
                             cudaStream_t st) {
  if (S <= 0) return 0;
  if (H < 16 || H % 16 || K < BKEYS || K % BKEYS || dq % 64 || dq > 576 || dv % 128 || dv > 512 || dv > dq || T < 1)
    return TB_ERR_ARG;
  SmlaParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.kv = reinterpret_cast<const __nv_bfloat16*>(kv);
  p.idx = idx;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse; p.teacher = teacher; p.sink = sink;
  p.S = S; p.H = H; p.T = T; p.K = K; p.dq = dq; p.dv = dv;
  p.hg = (H % 32 == 0) ? 32 : 16;
  p.teacher_atomic = (H / p.hg) > 1;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.stash = ((K / BKEYS) + dv / 128) * p.hg <= (int)TMEM_COLS ? 1 : 0;
  p.pipelined = g_sparse_mla_pipelined;
  p.status = status;
  return p.hg == 32 ? launch<32>(p, st) : launch<16>(p, st);
}
