// Dense bf16/fp16 GEMM on CTA PAIRS: tcgen05.mma.cta_group::2, 256 x 256 output tiles.
//
// Two CTAs of a 2-CTA cluster (the two SMs of a TPC) compute one 256 x 256 tile together.  Each CTA stages only
// ITS half of both operands (128 rows of A, 128 rows of B) with ordinary TMA loads and owns the 128 x 256 fp32
// accumulator of its rows in its own tensor memory; one thread of the leader CTA issues the MMAs for the pair
// and the tensor cores of both SMs read the two B halves from both shared memories.  Per SM and per k-block this
// moves (128 + 128) x 64 operands instead of (128 + 256) x 64 for the single-CTA 128 x 256 tile: two thirds of
// the L2 -> shared traffic and of the shared-memory fill for the same math, and a 32 KB stage, so the ring holds
// six stages where the single-CTA kernel holds four.
//
// Roles per CTA (192 threads): warp 0 TMA producer (its own operand halves; completion is counted on the
// LEADER's full barrier, which expects the bytes of both CTAs), warp 1 MMA issuer (leader only) and tensor-memory
// allocation, warps 2..5 epilogue (tcgen05.ld -> bf16 -> swizzled staging -> TMA store, or direct fp32 stores).
// Cross-CTA signals: the leader commits every consumed stage to the empty barrier of BOTH CTAs and every finished
// accumulator to the full-accumulator barrier of both; the epilogue warps of both CTAs arrive on the leader's
// accumulator-empty barrier (count 8).  Loads carry no cluster multicast: each CTA fetches what it needs itself.
//
// Tail waves: a persistent grid of P pairs over T tiles leaves the last wave partly empty whenever T mod P is
// small (4096 x 4096 x 8192: 256 tiles on 74 pairs = 3.46 waves).  The tiles of the last partial wave are
// therefore cut along the contraction into `split` equal parts that different pairs compute at the same time;
// every part adds its fp32 partial into a workspace with `red.global.add.f32`, and the part that arrives last
// (atomic ticket per tile) reads the sum back, converts and stores it, then clears the workspace for the next launch.
//
// Every wait is bounded (status word + abort flag, as in gemm_core.cuh).
#pragma once

#include "gemm_core.cuh"

namespace tbp {
using namespace tb;

constexpr int TM = 256, TN = 256;      // tile of the pair
constexpr int HM = 128, HN = 128;      // rows of A / rows of B staged per CTA
constexpr int BK = 64, UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_STAGE_BYTES = HM * BK * 2;   // 16 KB
constexpr int B_STAGE_BYTES = HN * BK * 2;   // 16 KB
constexpr int C_STAGE_BYTES = 32 * 1024;     // half of this CTA's 128 x 256 bf16 output
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + C_STAGE_BYTES + 1024 /*align*/ + 256;
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 192;
constexpr int MAX_SPLIT = 8;

struct PairParams {
  int M, N, K;
  int a_mn, b_mn;
  int out_fp32, is_bf16, accumulate, tma_store;
  long long ldc;
  void* C;
  int* status;
  // tail-wave split along the contraction
  int full_tiles;          // tiles [0, full_tiles) are computed whole; the rest in `split` parts each
  int split;               // 1 = no split
  float* ws;               // [tail tiles][256 x 256] fp32 partial sums, zero between launches
  unsigned int* tickets;   // [2 x tail tiles] arrival counters (one per CTA half), zero between launches
  int group_m;             // tile rows walked together (L2 reuse of the B panels)
  int stages;              // ring depth actually used (<= STAGES)
};

int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb_, const CUtensorMap& tc, const PairParams& p,
                int pairs, cudaStream_t st);
int max_pairs();

#ifdef TBP_DEFINE_KERNEL

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (a shared::cta address) in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion bytes are counted on a barrier that may live in the peer CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                   uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "mov.b64 da, {%1, %2};\n"
      "mov.b64 db, {%3, %4};\n"
      "setp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at `cluster_addr` once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

struct Unit {          // one piece of work of a pair: a tile, or one contraction slice of a tail tile
  int m0, n0;          // tile origin
  int kb0, kblocks;    // first 64-wide block and number of blocks
  int tail;            // index among the tail tiles, -1 for a whole tile
};

__device__ __forceinline__ int num_units(const PairParams& p, int tiles) {
  return p.full_tiles + (tiles - p.full_tiles) * p.split;
}

__device__ __forceinline__ Unit get_unit(const PairParams& p, int u) {
  const int num_m = (p.M + TM - 1) / TM, num_n = (p.N + TN - 1) / TN;
  const int kb_total = (p.K + BK - 1) / BK;
  Unit w;
  int t;
  if (u < p.full_tiles) {
    t = u; w.kb0 = 0; w.kblocks = kb_total; w.tail = -1;
  } else {
    const int r = u - p.full_tiles;
    w.tail = r / p.split;
    const int part = r - w.tail * p.split;
    t = p.full_tiles + w.tail;
    const int per = (kb_total + p.split - 1) / p.split;
    w.kb0 = part * per;
    w.kblocks = max(0, min(per, kb_total - w.kb0));
  }
  const int per_group = p.group_m * num_n;
  const int group = t / per_group, first_m = group * p.group_m;
  const int gsize = min(num_m - first_m, p.group_m);
  const int in_group = t - group * per_group;
  w.m0 = (first_m + in_group % gsize) * TM;
  w.n0 = (in_group / gsize) * TN;
  return w;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;
  uint8_t* smem_c = smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_c + C_STAGE_BYTES);
  uint64_t* full_bar = bars;                     // [STAGES]  used in the leader: bytes of both CTAs
  uint64_t* empty_bar = bars + STAGES;           // [STAGES]  one per CTA, signalled by the leader's commits
  uint64_t* tmem_full_bar = bars + 2 * STAGES;   // [2]       one per CTA, signalled by the leader's commits
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;  // [2]       used in the leader: 4 epilogue warps x 2 CTAs
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  volatile int* last_flag = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int pair = (int)blockIdx.x >> 1, npairs = (int)gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full_bar[a], 1); mbar_init(&tmem_empty_bar[a], 8); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_base_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers and tensor memory of BOTH CTAs exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const int tiles = ((p.M + TM - 1) / TM) * ((p.N + TN - 1) / TN);
  const int units = num_units(p, tiles);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs, own halves)
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int u = pair; u < units && ok; u += npairs) {
        const Unit w = get_unit(p, u);
        const int arow = w.m0 + (int)cta_rank * HM;   // this CTA's rows of A (and of the output)
        const int brow = w.n0 + (int)cta_rank * HN;   // this CTA's rows of B (columns of the output)
        for (int kb = 0; kb < w.kblocks; ++kb) {
          const int k0 = (w.kb0 + kb) * BK;
          if (!tbg::wait_bounded_relaxed(&empty_bar[stage], phase ^ 1, abort_flag, 64)) {
            if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_EMPTY); }
            ok = false; break;
          }
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * (A_STAGE_BYTES + B_STAGE_BYTES));
          const uint32_t fb = mapa(smem_u32(&full_bar[stage]), 0);
          uint8_t* sa = smem_a + stage * A_STAGE_BYTES;
          uint8_t* sb = smem_b + stage * B_STAGE_BYTES;
          if (!p.a_mn) {
            tma_load_2d_pair(sa, &tmap_a, fb, k0, arow);            // box {64 k, 128 m}
          } else {
#pragma unroll
            for (int j = 0; j < HM / 64; ++j)                        // box {64 m, 64 k}, 8 KB each
              tma_load_2d_pair(sa + j * 8192, &tmap_a, fb, arow + j * 64, k0);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sb, &tmap_b, fb, k0, brow);            // box {64 k, 128 n}
          } else {
#pragma unroll
            for (int j = 0; j < HN / 64; ++j)
              tma_load_2d_pair(sb + j * 8192, &tmap_b, fb, brow + j * 64, k0);
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      const uint32_t idesc = make_idesc_f16(TM, TN, p.is_bf16 != 0, p.a_mn != 0, p.b_mn != 0);
      // Descriptors of stage 0, k-step 0; everything that changes afterwards is the start-address field in the low
      // word.  K-major : rows of 128 B, 8-row swizzle atoms 1024 B apart (SBO); a K step of 16 elements = +32 B.
      // MN-major: 64-element (128 B) runs along M/N, K rows 128 B apart, 8-row atoms 1024 B apart (SBO), next
      //           64-wide M/N block 8192 B further (LBO); a K step of 16 rows = +2048 B.
      const uint64_t da0 = p.a_mn ? make_smem_desc(smem_u32(smem_a), 8192, 1024, 2)
                                  : make_smem_desc(smem_u32(smem_a), 16, 1024, 2);
      const uint64_t db0 = p.b_mn ? make_smem_desc(smem_u32(smem_b), 8192, 1024, 2)
                                  : make_smem_desc(smem_u32(smem_b), 16, 1024, 2);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
      const uint32_t a_k = p.a_mn ? (2048u >> 4) : (32u >> 4), b_k = p.b_mn ? (2048u >> 4) : (32u >> 4);
      const uint32_t a_k2 = 2 * a_k, a_k3 = 3 * a_k, b_k2 = 2 * b_k, b_k3 = 3 * b_k;
      // empty barriers of both CTAs as shared::cluster addresses (a CTA's window is linear: + 8 bytes per stage)
      const uint32_t eb0 = mapa(smem_u32(&empty_bar[0]), 0), eb1 = mapa(smem_u32(&empty_bar[0]), 1);
      int stage = 0; uint32_t phase = 0; bool ok = true;
      int acc = 0; uint32_t acc_phase = 0;
      for (int u = pair; u < units && ok; u += npairs) {
        const Unit w = get_unit(p, u);
        if (!tbg::wait_bounded(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag)) {
          if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_EMPTY); }
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        uint32_t accum = 0;   // the first MMA of a unit overwrites the accumulator
        for (int kb = 0; kb < w.kblocks; ++kb) {
          if (!tbg::wait_bounded(&full_bar[stage], phase, abort_flag)) {
            if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMA); }
            ok = false; break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + (uint32_t)stage * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + (uint32_t)stage * (B_STAGE_BYTES >> 4);
          umma_f16_pair_lohi(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, accum);
          umma_f16_pair_lohi(d_tmem, a_lo + a_k, a_hi, b_lo + b_k, b_hi, idesc, 1u);
          umma_f16_pair_lohi(d_tmem, a_lo + a_k2, a_hi, b_lo + b_k2, b_hi, idesc, 1u);
          umma_f16_pair_lohi(d_tmem, a_lo + a_k3, a_hi, b_lo + b_k3, b_hi, idesc, 1u);
          accum = 1u;
          umma_commit_pair(eb0 + (uint32_t)stage * 8u);
          umma_commit_pair(eb1 + (uint32_t)stage * 8u);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          const uint32_t tf = smem_u32(&tmem_full_bar[acc]);
          umma_commit_pair(mapa(tf, 0));
          umma_commit_pair(mapa(tf, 1));
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const bool issuer = warp == 2 && lane == 0;
    int acc = 0; uint32_t acc_phase = 0;
    for (int u = pair; u < units; u += npairs) {
      const Unit w = get_unit(p, u);
      bool ok = tbg::wait_bounded_relaxed(&tmem_full_bar[acc], acc_phase, abort_flag, 256);
      if (!ok && lane == 0 && *abort_flag == 0) {
        *abort_flag = 1;
        if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_FULL);
      }
      {
        uint32_t all_ok;
        asm volatile(
            "{\n"
            ".reg .pred pin, pout;\n"
            "setp.ne.u32 pin, %1, 0;\n"
            "barrier.red.and.pred pout, 1, 128, pin;\n"
            "selp.u32 %0, 1, 0, pout;\n"
            "}\n"
            : "=r"(all_ok)
            : "r"(ok ? 1u : 0u)
            : "memory");
        if (!all_ok) break;
      }
      tc_fence_after();
      const int row_in_tile = q * 32 + lane;            // row inside this CTA's half
      const int m_base = w.m0 + (int)cta_rank * HM;
      const int row = m_base + row_in_tile;
      const uint32_t taddr = tmem_base + acc * TN + ((uint32_t)(q * 32) << 16);
      const uint32_t tmem_empty_leader = mapa(smem_u32(&tmem_empty_bar[acc]), 0);
      bool finish = true;   // this unit writes the output (whole tile, or last arriving part of a tail tile)

      if (w.tail >= 0) {
        // add this part's fp32 partial into the tile's workspace; the last part to arrive finishes the tile
        float* wsrow = p.ws + ((long long)w.tail * TM + (int)cta_rank * HM + row_in_tile) * TN;
#pragma unroll 1
        for (int c = 0; c < TN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (w.kblocks > 0) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(wsrow + c * 32 + i),
                           "f"(__uint_as_float(r[i])), "f"(__uint_as_float(r[i + 1])),
                           "f"(__uint_as_float(r[i + 2])), "f"(__uint_as_float(r[i + 3]))
                           : "memory");
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(tmem_empty_leader);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (issuer) {
          // one ticket per CTA half: 2 * split arrivals complete a tile
          const unsigned int t = atomicAdd(p.tickets + 2 * w.tail + cta_rank, 1u);
          *last_flag = (t == (unsigned int)p.split - 1u) ? 1 : 0;
          if (*last_flag) p.tickets[2 * w.tail + cta_rank] = 0;  // ready for the next launch
          __threadfence();
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        finish = *last_flag != 0;
      }

      if (!finish) {
        // nothing to store for this unit
      } else if (p.tma_store) {
        // half-tile -> swizzled shared staging (two halves of 128 columns) -> TMA store (clipped at the edges)
        const uint32_t srow = smem_u32(smem_c) + row_in_tile * 128;
        float* wsrow = w.tail >= 0 ? p.ws + ((long long)w.tail * TM + (int)cta_rank * HM + row_in_tile) * TN : nullptr;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          if (issuer) tma_store_wait_read<0>();
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t r[32];
            if (w.tail < 0) {
              tmem_ld_32x32(taddr + (half * 4 + cc) * 32, r);
              tmem_ld_wait();
            } else {
              float4* src = reinterpret_cast<float4*>(wsrow + (half * 4 + cc) * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 v = __ldcg(src + i);
                r[4 * i] = __float_as_uint(v.x); r[4 * i + 1] = __float_as_uint(v.y);
                r[4 * i + 2] = __float_as_uint(v.z); r[4 * i + 3] = __float_as_uint(v.w);
                __stcg(src + i, make_float4(0.f, 0.f, 0.f, 0.f));  // workspace is zero again for the next launch
              }
            }
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float lo = __uint_as_float(r[2 * i]), hi = __uint_as_float(r[2 * i + 1]);
              if (p.is_bf16) {
                pk[i] = pack_bf16x2(lo, hi);
              } else {
                __half2 h = __floats2half2_rn(lo, hi);
                pk[i] = *reinterpret_cast<uint32_t*>(&h);
              }
            }
            const uint32_t box = srow + (cc >> 1) * 16384;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t chunk = (uint32_t)((cc & 1) * 4 + i) ^ (uint32_t)(row_in_tile & 7);  // 128B swizzle
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(box + chunk * 16), "r"(pk[4 * i]),
                           "r"(pk[4 * i + 1]), "r"(pk[4 * i + 2]), "r"(pk[4 * i + 3])
                           : "memory");
            }
          }
          if (half == 1 && w.tail < 0) {  // all TMEM reads of this accumulator are done
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(tmem_empty_leader);
          }
          fence_proxy_async();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (issuer) {
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              const int x = w.n0 + half * 128 + b * 64;
              if (x >= p.N || m_base >= p.M) continue;
              tma_store_2d(&tmap_c, smem_c + b * 16384, x, m_base);
            }
            tma_store_commit();
          }
        }
      } else {
        tbg::GemmParams gp;  // only the fields store_row32 reads
        gp.out_fp32 = p.out_fp32; gp.is_bf16 = p.is_bf16; gp.accumulate = p.accumulate;
        float* wsrow = w.tail >= 0 ? p.ws + ((long long)w.tail * TM + (int)cta_rank * HM + row_in_tile) * TN : nullptr;
#pragma unroll 1
        for (int c = 0; c < TN / 32; ++c) {
          uint32_t r[32];
          if (w.tail < 0) {
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
          } else {
            float4* src = reinterpret_cast<float4*>(wsrow + c * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 v = __ldcg(src + i);
              r[4 * i] = __float_as_uint(v.x); r[4 * i + 1] = __float_as_uint(v.y);
              r[4 * i + 2] = __float_as_uint(v.z); r[4 * i + 3] = __float_as_uint(v.w);
              __stcg(src + i, make_float4(0.f, 0.f, 0.f, 0.f));
            }
          }
          const int col = w.n0 + c * 32;
          if (row < p.M && col < p.N) tbg::store_row32(gp, p.C, p.ldc, row, col, p.N, r);
        }
        if (w.tail < 0) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(tmem_empty_leader);
        }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (issuer && p.tma_store) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer may still signal this CTA's barriers or read its shared memory until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

int max_pairs() {
  static int cached = 0;
  if (cached) return cached;
  int n = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 74, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  if (cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
      cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel, &cfg) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    n = tbg::sm_count() / 2;
  }
  const int by_sm = tbg::sm_count() / 2;
  cached = n < by_sm ? n : by_sm;
  if (cached < 1) cached = 1;
  return cached;
}

int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb_, const CUtensorMap& tc, const PairParams& p,
                int pairs, cudaStream_t st) {
  TB_CUDA_CHECK(cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  gemm_pair_kernel<<<2 * pairs, NUM_THREADS, SMEM_BYTES, st>>>(ta, tb_, tc, p);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
#endif  // TBP_DEFINE_KERNEL

}  // namespace tbp
