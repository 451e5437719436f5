// Core of the tcgen05 GEMM family: one persistent, warp-specialised kernel, several tile schedulers.
//
//   C = A · B with bf16/fp16 operands and fp32 accumulation in tensor memory.
//
// Roles (192 threads, one CTA per SM):
//   warp 0      TMA producer: global (local or peer) → 128B-swizzled shared tiles, 4-stage mbarrier ring
//   warp 1      MMA issuer : one thread issues tcgen05.mma 128x256x16; two TMEM accumulator buffers
//   warps 2..5  epilogue   : tcgen05.ld → convert → global (local memory or a peer's staging buffer)
//
// Schedulers (`GemmParams::mode`):
//   PLAIN      dense [M,N,K]
//   GROUPED_M  rows of A/C are grouped (MoE experts): group g owns rows [offs[g-1], offs[g]), every
//              boundary a multiple of 128 (padded layout), B holds one matrix per group
//   GROUPED_K  weight gradient of GROUPED_M: C[g] = A_gᵀ · B_g, the contraction runs over the rows of group g
//   ALLGATHER  A is sharded by rows over `nranks` GPUs; each M tile is TMA-loaded straight from the
//              owner's memory (no multicast) once that owner's ready flag has arrived
//   ALLGATHER_B same for a B operand sharded by rows of N (FSDP weight shards gathered inside the GEMM);
//              `n_shard` rows per rank, a multiple of 256
//   INDEXER    lightning-indexer scores: rows of A are index KEYS, rows of B are (query, head) pairs, so a thread of
//              the epilogue (one TMEM lane = one key) holds all heads of its queries and computes
//              Σ_head w[q,head]·relu(acc) without any exchange; fp32 scores [query, key]; tiles that lie
//              entirely in the causal future of their queries are skipped by every role
//   SCATTER    C is reduce-scattered by rows: each tile is stored into the owner rank's staging slot
//              for this rank; the last tile for an owner releases a flag on that owner
//   SCATTER_N  projection fused with a head -> sequence all-to-all (Ulysses): columns of C belong to the rank that
//              owns those heads; every 64-column box is stored into that rank's receive buffer
//              [batch * seq_full, n_shard] at the rows of this rank's sequence slice
//   GATHER_K   the reverse exchange fused into the consuming GEMM: the contraction dimension of A is sliced by
//              owner rank (k_shard columns each, rows laid out [batch * seq_full] on the owner); copier CTAs bring
//              the remote slices of this rank's rows into a local [nranks][M][k_shard] buffer once
//
// Operand storage: a_mn/b_mn = 0 → K-major ([M,K] / [N,K] row-major), 1 → MN-major ([K,M] / [K,N]).
// Every wait is time-bounded; on expiry the kernel records a status code, raises a CTA-wide abort flag,
// drains and frees its tensor memory.
#pragma once

#include "../common/tb_common.cuh"

namespace tbg {
using namespace tb;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int MAX_GROUPS = 256;
constexpr int MAX_RANKS = 8;
constexpr int C_STAGE_BYTES = 32 * 1024;    // epilogue staging: half an output tile (128 x 128 x 2 B)
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + C_STAGE_BYTES + 1024 /*align*/ +
                           256 /*barriers*/ + (MAX_GROUPS + 1) * 4;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 16;
constexpr int NUM_THREADS = 192;
constexpr unsigned long long WAIT_NS = 2000000000ull;

enum Mode : int {
  PLAIN = 0, GROUPED_M = 1, GROUPED_K = 2, ALLGATHER = 3, SCATTER = 4, ALLGATHER_B = 5, INDEXER = 6, SCATTER_N = 7,
  GATHER_K = 8
};

struct GemmParams {
  int mode;
  int M, N, K;        // PLAIN/ALLGATHER/SCATTER: full problem. GROUPED_M: M = row capacity. GROUPED_K: M,N = per-group output
  int a_mn, b_mn;
  int out_fp32, is_bf16, accumulate;
  long long ldc;
  void* C;
  int* status;
  // grouped
  int num_groups;
  const int* offs;          // [num_groups] cumulative (padded) row ends, device memory
  long long b_group_rows;   // rows of B's 2-D view per group (N for K-major B, K for MN-major B)
  long long c_group_stride; // GROUPED_K: elements between consecutive C[g]
  // collectives
  int rank, nranks;
  int m_shard;              // rows per rank (multiple of 128)
  int n_shard;              // ALLGATHER_B: rows of B per rank (multiple of 256); SCATTER_N: columns of C per owner
  int k_shard;              // GATHER_K: contraction columns per owner (multiple of 64)
  int seq_local, seq_full;  // SCATTER_N / GATHER_K: local row b*seq_local+s is row b*seq_full+rank*seq_local+s there
  const unsigned int* ready_flags;  // ALLGATHER: [nranks] in local memory, written by peers
  unsigned int epoch;
  void* stage_ptrs[MAX_RANKS];          // SCATTER: staging buffer base on every rank: [src][m_shard][N]
  unsigned int* peer_flags[MAX_RANKS];  // SCATTER: flag array [nranks] on every rank (slot = source rank)
  unsigned int* tile_counters;          // SCATTER: [nranks] local counters of finished tiles per owner
  int tma_store;                        // epilogue stores whole tiles with TMA (16-bit output, no accumulate)
  // gather modes: copier CTAs bring every remote shard into `gather_dst` exactly once
  const void* peer_src[MAX_RANKS];      // shard base on every rank (peer-mapped)
  void* gather_dst;                     // local [nranks * shard_rows, K] buffer
  unsigned int* chunk_flags;            // local [num chunks]; chunk c holds `epoch` once it has been copied
  int num_copiers;
  // INDEXER
  const float* idx_weights;  // [N] = [queries * heads] head weights (already scaled)
  int idx_heads;             // heads per query (a power of two, at most 256)
  float* idx_scores;         // [queries, idx_ld] fp32 out
  long long idx_ld;
  int idx_pos_offset;        // key t is visible to local query s iff t < (idx_pos_offset + s + 1) / idx_ratio
  int idx_ratio;             // 1 = plain causal keys; r > 1 = keys are blocks of r tokens, visible once closed
};

struct CMaps {
  CUtensorMap m[MAX_RANKS];
};

struct AMaps {
  CUtensorMap m[MAX_RANKS];
};

struct Tile {
  int valid;
  int m0, n0;        // output coordinates (GROUPED_K: within the group's matrix)
  int a_row;         // row (K-major A) or column (MN-major A) coordinate of the A tile in its tensor map
  int src;           // which A map
  long long b_off;   // row offset into B's 2-D view
  int k0, kblocks;   // contraction start (elements) and number of 64-wide blocks
  int row_end;       // stores are masked to rows < row_end
  int group;
  int chunk;         // gather modes: index of the gathered operand's tile row (copier hand-off flag)
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded waits read the global timer only after a stretch of failed polls: a %globaltimer read costs on the order
// of a microsecond, and short-K tiles block on four barriers per tile (reading it on entry of every blocked wait
// made the tile loop handoff-bound: 8.6 us per 128x256x128 tile against 0.55 us of MMA).
__device__ __forceinline__ bool wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;
  uint32_t it = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 1023u) == 0u) {
      if (*abort_flag != 0) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_NS) return false;
    }
  }
}

// Same wait for the roles that are NOT on the critical path of MMA issue (epilogue warps waiting for a finished
// accumulator, the TMA producer waiting for a free stage).  Such a warp shares its scheduler with the MMA-issuing
// warp or the producer; a hot polling loop would take issue slots from them, so it sleeps between polls.
__device__ __forceinline__ bool wait_bounded_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                     unsigned sleep_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;
  uint32_t it = 0;
  while (true) {
    __nanosleep(sleep_ns);
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 255u) == 0u) {
      if (*abort_flag != 0) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_NS) return false;
    }
  }
}

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded spin on a flag written by a peer GPU
__device__ __forceinline__ bool wait_flag_ge(const unsigned int* flag, unsigned int want, volatile int* abort_flag) {
  if ((int)(ld_acquire_sys(flag) - want) >= 0) return true;
  unsigned long long t0 = 0;
  uint32_t it = 0;
  while (true) {
    if ((int)(ld_acquire_sys(flag) - want) >= 0) return true;
    if ((++it & 63u) == 0u) {
      if (abort_flag != nullptr && *abort_flag != 0) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_NS) return false;
    }
  }
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded spin on a flag written by another CTA of this GPU
__device__ __forceinline__ bool wait_local_flag_ge(const unsigned int* flag, unsigned int want,
                                                   volatile int* abort_flag) {
  if ((int)(ld_acquire_gpu(flag) - want) >= 0) return true;
  unsigned long long t0 = 0;
  uint32_t it = 0;
  while (true) {
    if ((int)(ld_acquire_gpu(flag) - want) >= 0) return true;
    if ((++it & 63u) == 0u) {
      if (abort_flag != nullptr && *abort_flag != 0) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_NS) return false;
    }
  }
}

// INDEXER: the whole tile is in the causal future of all of its queries (nothing to compute or store)
__device__ __forceinline__ bool tile_is_future(const GemmParams& p, int m0, int n0) {
  if (p.mode != INDEXER) return false;
  const int last_query = (min(n0 + BN, p.N) - 1) / p.idx_heads;  // columns are (query, head) pairs
  return m0 >= (p.idx_pos_offset + last_query + 1) / p.idx_ratio;  // rows are keys
}

__device__ __forceinline__ int total_tiles(const GemmParams& p, const int* s_offs) {
  const int num_n = (p.N + BN - 1) / BN;
  if (p.mode == GROUPED_M) return (s_offs[p.num_groups] / BM) * num_n;
  if (p.mode == GROUPED_K) return p.num_groups * ((p.M + BM - 1) / BM) * num_n;
  return ((p.M + BM - 1) / BM) * num_n;
}

// s_offs: [num_groups + 1] with s_offs[0] = 0 (shared memory copy of the cumulative offsets)
__device__ __forceinline__ Tile get_tile(const GemmParams& p, const int* s_offs, int t) {
  Tile tl;
  tl.valid = 1; tl.src = 0; tl.chunk = 0; tl.b_off = 0; tl.k0 = 0; tl.kblocks = (p.K + BK - 1) / BK; tl.group = 0;
  const int num_n = (p.N + BN - 1) / BN;
  if (p.mode == GROUPED_M) {
    const int mt = t / num_n, nt = t - mt * num_n;
    tl.m0 = mt * BM; tl.n0 = nt * BN; tl.a_row = tl.m0;
    int g = 0;
    while (g < p.num_groups - 1 && s_offs[g + 1] <= tl.m0) ++g;
    tl.group = g; tl.b_off = (long long)g * p.b_group_rows; tl.row_end = s_offs[g + 1];
    return tl;
  }
  if (p.mode == GROUPED_K) {
    const int num_m = (p.M + BM - 1) / BM;
    const int per = num_m * num_n;
    const int g = t / per, r = t - g * per;
    const int mt = r / num_n, nt = r - mt * num_n;
    tl.group = g; tl.m0 = mt * BM; tl.n0 = nt * BN; tl.a_row = tl.m0; tl.row_end = p.M;
    tl.k0 = s_offs[g]; tl.kblocks = (s_offs[g + 1] - s_offs[g] + BK - 1) / BK;
    return tl;
  }
  const int num_m = (p.M + BM - 1) / BM;
  int mt, nt;
  {
    const int per_group = GROUP_M * num_n;
    const int group = t / per_group, first_m = group * GROUP_M;
    const int gsize = min(num_m - first_m, GROUP_M);
    const int in_group = t - group * per_group;
    mt = first_m + in_group % gsize; nt = in_group / gsize;
  }
  if (p.mode == ALLGATHER) {
    // start with the local shard, then walk the peers in ring order: spreads link load, hides flag latency
    const int per = p.m_shard / BM;
    mt = (mt + p.rank * per) % num_m;
    tl.src = (mt * BM) / p.m_shard;
    // own shard: read in place (map 0); remote shards: read the local gathered copy (map 1, global rows)
    tl.a_row = tl.src == p.rank ? mt * BM - tl.src * p.m_shard : mt * BM;
    tl.chunk = mt;
  } else if (p.mode == ALLGATHER_B) {
    const int per = p.n_shard / BN;
    const int num_nt = (p.N + BN - 1) / BN;
    nt = (nt + p.rank * per) % num_nt;
    tl.src = (nt * BN) / p.n_shard;
    tl.b_off = tl.src == p.rank ? -(long long)tl.src * p.n_shard : 0;  // own shard in place, else gathered copy
    tl.chunk = nt;
    tl.a_row = mt * BM;
  } else if (p.mode == SCATTER) {
    // tiles owned by this rank come last (they need no transfer)
    const int per = p.m_shard / BM;
    mt = (mt + ((p.rank + 1) % p.nranks) * per) % num_m;
    tl.a_row = mt * BM;
  } else if (p.mode == SCATTER_N) {
    // start at the next rank's columns, finish with the local ones
    nt = (nt + (((p.rank + 1) % p.nranks) * p.n_shard) / BN) % num_n;
    tl.a_row = mt * BM;
  } else {
    tl.a_row = mt * BM;
  }
  tl.m0 = mt * BM; tl.n0 = nt * BN; tl.row_end = p.M;
  return tl;
}

// SCATTER_N / GATHER_K: row of the full-sequence layout that holds local row `m` of rank `rank`
__device__ __forceinline__ int seq_row(const GemmParams& p, int m, int rank) {
  const int b = m / p.seq_local;
  return b * p.seq_full + rank * p.seq_local + (m - b * p.seq_local);
}

// store 32 consecutive fp32 accumulator values of one row
__device__ __forceinline__ void store_row32(const GemmParams& p, void* base, long long ld, int row, int col,
                                            int ncols_total, const uint32_t (&r)[32]) {
  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(base) + (long long)row * ld + col;
    if (col + 32 <= ncols_total) {
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
      for (int i = 0; i < 32 && col + i < ncols_total; ++i)
        dst[i] = __uint_as_float(r[i]) + (p.accumulate ? dst[i] : 0.f);
    }
  } else if (p.is_bf16) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(base) + (long long)row * ld + col;
    if (col + 32 <= ncols_total) {
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
        *reinterpret_cast<uint4*>(dst + i) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                                        pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
      }
    } else {
      for (int i = 0; i < 32 && col + i < ncols_total; ++i)
        dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]) + (p.accumulate ? __bfloat162float(dst[i]) : 0.f));
    }
  } else {
    __half* dst = reinterpret_cast<__half*>(base) + (long long)row * ld + col;
    for (int i = 0; i < 32 && col + i < ncols_total; ++i)
      dst[i] = __float2half_rn(__uint_as_float(r[i]) + (p.accumulate ? __half2float(dst[i]) : 0.f));
  }
}

}  // namespace tbg
