// The kernel body shared by every GEMM entry point (see gemm_core.cuh for the design).
#pragma once

#include "gemm_core.cuh"

namespace tbg {

// The kernel is compiled once (in gemm_bf16.cu, which defines TBG_DEFINE_KERNEL); other files call launch().
int launch(const AMaps& am, const CUtensorMap& tb_, const CMaps& cm, const GemmParams& p, int grid, cudaStream_t st);

#ifdef TBG_DEFINE_KERNEL

// Copier role of the gather modes: pull remote shards into local memory once, chunk by chunk, and hand each
// chunk to the GEMM CTAs through a local flag.  Chunks are visited in ring order starting at the next rank.
// One thread drives bulk asynchronous copies (peer global -> shared -> local global) through a ring of
// COPY_BUFS shared buffers, so a CTA keeps ~190 KB in flight on the link without spending registers or
// issue slots; no multicast is involved.  A copier owns whole chunks (one completion flag per chunk, not per piece).
constexpr int COPY_PIECE = 32 * 1024;
constexpr int COPY_BUFS = 6;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void copier_role(const GemmParams& p, uint8_t* bufs, uint64_t* bars,
                                            volatile int* abort_flag) {
  if (threadIdx.x != 0) return;
  for (int b = 0; b < COPY_BUFS; ++b) mbar_init(&bars[b], 1);
  fence_barrier_init();
  // GATHER_K: a chunk is 128 rows of one owner's k_shard-wide slice (contiguous on the owner); chunks are visited
  // row-block by row-block, since every output tile needs the slices of all owners for its rows.
  const bool gk = p.mode == GATHER_K;
  const int chunk_rows = p.mode == ALLGATHER_B ? BN : BM;
  const int shard_rows = gk ? p.M : (p.mode == ALLGATHER ? p.m_shard : p.n_shard);
  const int per = shard_rows / chunk_rows;
  const int remote_chunks = (p.nranks - 1) * per;
  const long long row_bytes = (long long)(gk ? p.k_shard : p.K) * 2;
  const long long chunk_bytes = (long long)chunk_rows * row_bytes;
  const int pieces = (int)((chunk_bytes + COPY_PIECE - 1) / COPY_PIECE);
  int my_chunks = 0;
  for (int idx = blockIdx.x; idx < remote_chunks; idx += p.num_copiers) ++my_chunks;
  const long long total = (long long)my_chunks * pieces;
  unsigned int seen = 1u << p.rank;
  const int D = COPY_BUFS - 1;  // loads run this many pieces ahead of the stores
  auto locate = [&](int idx, int& src, int& within, long long& src_off) {
    int d;
    if (gk) { within = idx / (p.nranks - 1); d = idx - within * (p.nranks - 1) + 1; }
    else { d = idx / per + 1; within = idx - (d - 1) * per; }
    src = (p.rank + d) % p.nranks;
    src_off = gk ? (long long)seq_row(p, within * BM, p.rank) * row_bytes : (long long)within * chunk_bytes;
  };
  for (long long i = 0; i < total + D; ++i) {
    if (i < total) {
      const int ci = (int)(i / pieces), pi = (int)(i - (long long)ci * pieces);
      int src, within; long long src_off;
      locate(blockIdx.x + ci * p.num_copiers, src, within, src_off);
      if (!(seen & (1u << src))) {
        if (!wait_flag_ge(p.ready_flags + src, p.epoch, abort_flag)) {
          if (p.status) atomicExch(p.status, TB_ERR_WAIT_PEER);
          return;  // GEMM CTAs time out on the chunk flag and report as well
        }
        seen |= 1u << src;
      }
      const int b = (int)(i % COPY_BUFS);
      if (i >= COPY_BUFS) tma_store_wait_read<0>();  // the store that used this buffer has read it
      const long long off = (long long)pi * COPY_PIECE;
      const uint32_t bytes = (uint32_t)((chunk_bytes - off) < COPY_PIECE ? (chunk_bytes - off) : COPY_PIECE);
      const uint8_t* from = reinterpret_cast<const uint8_t*>(p.peer_src[src]) + src_off + off;
      mbar_expect_tx(&bars[b], bytes);
      bulk_load(bufs + b * COPY_PIECE, from, bytes, &bars[b]);
    }
    const long long j = i - D;
    if (j >= 0 && j < total) {
      const int ci = (int)(j / pieces), pi = (int)(j - (long long)ci * pieces);
      int src, within; long long src_off;
      locate(blockIdx.x + ci * p.num_copiers, src, within, src_off);
      const int b = (int)(j % COPY_BUFS);
      if (!wait_bounded(&bars[b], (uint32_t)((j / COPY_BUFS) & 1), abort_flag)) {
        if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMA);
        return;
      }
      const long long off = (long long)pi * COPY_PIECE;
      const uint32_t bytes = (uint32_t)((chunk_bytes - off) < COPY_PIECE ? (chunk_bytes - off) : COPY_PIECE);
      uint8_t* to = reinterpret_cast<uint8_t*>(p.gather_dst) + ((long long)src * per + within) * chunk_bytes + off;
      bulk_store(to, bufs + b * COPY_PIECE, bytes);
      tma_store_commit();
      if (pi == pieces - 1) {  // chunk complete: make it visible, then hand it to the GEMM CTAs
        tma_store_wait_all<0>();
        __threadfence();
        st_release_gpu(p.chunk_flags + src * per + within, p.epoch);
      }
    }
  }
  tma_store_wait_all<0>();
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ AMaps amaps, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CMaps cmaps, const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;
  uint8_t* smem_c = smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);  // 32 KB, 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_c + C_STAGE_BYTES);
  uint64_t* full_bar = bars;                     // [STAGES]
  uint64_t* empty_bar = bars + STAGES;           // [STAGES]
  uint64_t* tmem_full_bar = bars + 2 * STAGES;   // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;  // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  int* s_offs = reinterpret_cast<int*>(bars) + 64;  // 256 B after the barrier block: [num_groups + 1]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool gather_mn = p.mode == ALLGATHER || p.mode == ALLGATHER_B;  // whole tiles of A / B come from one owner
  const bool gather_k = p.mode == GATHER_K;                              // the owner changes along the contraction
  const bool gather = gather_mn || gather_k;

  if (gather && (int)blockIdx.x < p.num_copiers) {
    if (threadIdx.x == 0) *abort_flag = 0;
    __syncthreads();
    copier_role(p, smem_a, bars, abort_flag);  // the operand stages double as copy buffers here
    return;
  }
  const int cta = gather ? (int)blockIdx.x - p.num_copiers : (int)blockIdx.x;
  const int ncta = gather ? (int)gridDim.x - p.num_copiers : (int)gridDim.x;

  if (p.mode == GROUPED_M || p.mode == GROUPED_K) {
    for (int i = threadIdx.x; i <= p.num_groups; i += NUM_THREADS) s_offs[i] = i == 0 ? 0 : p.offs[i - 1];
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full_bar[a], 1); mbar_init(&tmem_empty_bar[a], 4); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const int num_tiles = total_tiles(p, s_offs);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += ncta) {
        const Tile tl = get_tile(p, s_offs, t);
        if (tile_is_future(p, tl.m0, tl.n0)) continue;
        int gmap = 0;  // which map of the gathered operand: 0 = own shard in place, 1 = local gathered copy
        if (gather_mn && tl.src != p.rank) {
          if (!wait_local_flag_ge(p.chunk_flags + tl.chunk, p.epoch, abort_flag)) {
            if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_PEER); }
            break;
          }
          // the chunk was written with ordinary stores by a copier CTA; TMA reads through the async proxy
          asm volatile("fence.proxy.async.global;" ::: "memory");
          gmap = 1;
        }
        const CUtensorMap* ta = p.mode == ALLGATHER_B ? &tmap_b : &amaps.m[p.mode == ALLGATHER ? gmap : 0];
        const CUtensorMap* tbm = p.mode == ALLGATHER_B ? &amaps.m[gmap] : &tmap_b;
        const int kps = gather_k ? p.k_shard / BK : 1;  // 64-wide blocks per owner slice
        for (int kb = 0; kb < tl.kblocks; ++kb) {
          int k0 = tl.k0 + kb * BK;  // contraction coordinate (the B operand always uses it)
          int ax = k0, ay = tl.a_row;
          if (gather_k) {
            // own slice first, then the owners in ring order (the order in which the copiers fetch them)
            const int s = (p.rank + kb / kps) % p.nranks, kk = kb - (kb / kps) * kps;
            k0 = s * p.k_shard + kk * BK;
            ax = kk * BK;
            if (s == p.rank) {
              ta = &amaps.m[0];  // own slice in place: rows of the full-sequence layout
              ay = seq_row(p, tl.m0, p.rank);
            } else {
              if (kk == 0) {
                if (!wait_local_flag_ge(p.chunk_flags + s * (p.M / BM) + tl.m0 / BM, p.epoch, abort_flag)) {
                  if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_PEER); }
                  ok = false; break;
                }
                asm volatile("fence.proxy.async.global;" ::: "memory");
              }
              ta = &amaps.m[1];  // local copy [owner][M][k_shard]
              ay = s * p.M + tl.m0;
            }
          }
          if (!wait_bounded_relaxed(&empty_bar[stage], phase ^ 1, abort_flag, 64)) {
            if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_EMPTY); }
            ok = false; break;
          }
          mbar_expect_tx(&full_bar[stage], A_STAGE_BYTES + B_STAGE_BYTES);
          uint8_t* sa = smem_a + stage * A_STAGE_BYTES;
          uint8_t* sb = smem_b + stage * B_STAGE_BYTES;
          if (!p.a_mn) {
            tma_load_2d(sa, ta, &full_bar[stage], ax, ay);  // box {64 k, 128 m}
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)  // box {64 m, 64 k}, 8 KB each
              tma_load_2d(sa + j * 8192, ta, &full_bar[stage], tl.a_row + j * 64, k0);
          }
          if (!p.b_mn) {
            tma_load_2d(sb, tbm, &full_bar[stage], k0, (int)(tl.b_off + tl.n0));  // box {64 k, 256 n}
          } else {
            const int krow = p.mode == GROUPED_K ? k0 : (int)(tl.b_off + k0);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, tbm, &full_bar[stage], tl.n0 + j * 64, krow);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(BM, BN, p.is_bf16 != 0, p.a_mn != 0, p.b_mn != 0);
      // Descriptors of stage 0, k-step 0.  This thread is alone on its warp: every instruction between two MMAs
      // delays the next one, so the loop only adds stage / k offsets to the start-address field (low word).
      // K-major : rows of 128 B, 8-row swizzle atoms 1024 B apart (SBO); a K step of 16 elements = +32 B
      // MN-major: 64-element (128 B) runs along M/N, K rows 128 B apart, 8-row atoms 1024 B apart (SBO),
      //           next 64-wide M/N block 8192 B further (LBO); a K step of 16 rows = +2048 B
      const uint64_t da0 = p.a_mn ? make_smem_desc(smem_u32(smem_a), 8192, 1024, 2)
                                  : make_smem_desc(smem_u32(smem_a), 16, 1024, 2);
      const uint64_t db0 = p.b_mn ? make_smem_desc(smem_u32(smem_b), 8192, 1024, 2)
                                  : make_smem_desc(smem_u32(smem_b), 16, 1024, 2);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
      const uint32_t a_k = p.a_mn ? (2048u >> 4) : (32u >> 4), b_k = p.b_mn ? (2048u >> 4) : (32u >> 4);
      int stage = 0; uint32_t phase = 0; bool ok = true;
      int acc = 0; uint32_t acc_phase = 0;
      for (int t = cta; t < num_tiles && ok; t += ncta) {
        const Tile tl = get_tile(p, s_offs, t);
        if (tile_is_future(p, tl.m0, tl.n0)) continue;
        if (!wait_bounded(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag)) {
          if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_EMPTY); }
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t accum = 0;  // the first MMA of a tile overwrites the accumulator
        for (int kb = 0; kb < tl.kblocks; ++kb) {
          if (!wait_bounded(&full_bar[stage], phase, abort_flag)) {
            if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMA); }
            ok = false; break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + (uint32_t)stage * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + (uint32_t)stage * (B_STAGE_BYTES >> 4);
          umma_f16_lohi(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, accum);
          umma_f16_lohi(d_tmem, a_lo + a_k, a_hi, b_lo + b_k, b_hi, idesc, 1u);
          umma_f16_lohi(d_tmem, a_lo + 2 * a_k, a_hi, b_lo + 2 * b_k, b_hi, idesc, 1u);
          umma_f16_lohi(d_tmem, a_lo + 3 * a_k, a_hi, b_lo + 3 * b_k, b_hi, idesc, 1u);
          accum = 1u;
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full_bar[acc]);  // with no MMA issued (empty group) this arrives at once
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const bool issuer = warp == 2 && lane == 0;
    int acc = 0; uint32_t acc_phase = 0;
    for (int t = cta; t < num_tiles; t += ncta) {
      const Tile tl = get_tile(p, s_offs, t);
      if (tile_is_future(p, tl.m0, tl.n0)) continue;
      bool ok = wait_bounded_relaxed(&tmem_full_bar[acc], acc_phase, abort_flag, 256);
      if (!ok && lane == 0 && *abort_flag == 0) {
        *abort_flag = 1;
        if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_FULL);
      }
      {
        // one decision for all four epilogue warps: they share named barriers further down
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
      const int row_in_tile = q * 32 + lane;
      const int row = tl.m0 + row_in_tile;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      int dst_rank = 0;
      if (p.mode == SCATTER) dst_rank = tl.m0 / p.m_shard;

      if (p.mode == INDEXER) {
        // score[q, t] = Σ_h w[q, h] · relu(acc[t, (q, h)]): rows of the tile are KEYS (one per TMEM lane = per
        // thread), columns are (query, head) pairs, so the head sum runs inside a thread with no exchange at all;
        // for a fixed query the 128 threads store 128 consecutive keys (coalesced).
        float* wst = reinterpret_cast<float*>(smem_c);  // weights of this tile's 256 columns (broadcast reads)
        const int hmask = p.idx_heads - 1;              // heads is a power of two
        const int hshift = 31 - __clz(p.idx_heads);
        const int et = (warp - 2) * 32 + lane;          // 0..127 among the epilogue threads
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the previous tile's readers are done with wst
        for (int i = et; i < BN; i += 128) wst[i] = (tl.n0 + i) < p.N ? p.idx_weights[tl.n0 + i] : 0.f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int queries = p.N >> hshift;
        if (p.idx_heads >= 32) {
          // A query's heads end on 32-column chunk boundaries.  One epilogue warp runs alone on its scheduler, so
          // the loop is written for latency: four independent accumulators, weights as 128-bit shared loads, the
          // next chunk's tcgen05.ld in flight while this one is summed, one boundary test per chunk.
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
          uint32_t r[2][32];
          tmem_ld_32x32(taddr, r[0]);
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) {
            tmem_ld_wait();
            if (c + 1 < BN / 32) tmem_ld_32x32(taddr + (c + 1) * 32, r[(c + 1) & 1]);
            const float4* w4 = reinterpret_cast<const float4*>(wst + c * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 w = w4[i];
              s0 = fmaf(fmaxf(__uint_as_float(r[c & 1][4 * i + 0]), 0.f), w.x, s0);
              s1 = fmaf(fmaxf(__uint_as_float(r[c & 1][4 * i + 1]), 0.f), w.y, s1);
              s2 = fmaf(fmaxf(__uint_as_float(r[c & 1][4 * i + 2]), 0.f), w.z, s2);
              s3 = fmaf(fmaxf(__uint_as_float(r[c & 1][4 * i + 3]), 0.f), w.w, s3);
            }
            if ((((c + 1) * 32) & hmask) == 0) {  // last head of a query
              const int query = (tl.n0 + c * 32) >> hshift;
              if (row < p.M && query < queries)
                p.idx_scores[(long long)query * p.idx_ld + row] = (s0 + s1) + (s2 + s3);
              s0 = s1 = s2 = s3 = 0.f;
            }
          }
        } else {
          float sum = 0.f;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              sum = fmaf(fmaxf(__uint_as_float(r[i]), 0.f), wst[c * 32 + i], sum);
              if (((c * 32 + i + 1) & hmask) == 0) {  // last head of a query
                const int query = (tl.n0 + c * 32 + i) >> hshift;
                if (row < p.M && query < queries) p.idx_scores[(long long)query * p.idx_ld + row] = sum;
                sum = 0.f;
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
      } else if (p.tma_store) {
        // tile → swizzled shared staging (two halves of 128 columns) → TMA store (coalesced, clipped at edges)
        const CUtensorMap* cm = &cmaps.m[p.mode == SCATTER ? dst_rank : 0];
        int y = tl.m0;
        if (p.mode == GROUPED_K) y = tl.group * p.M + tl.m0;
        else if (p.mode == SCATTER) y = p.rank * p.m_shard + (tl.m0 - dst_rank * p.m_shard);
        else if (p.mode == SCATTER_N) y = seq_row(p, tl.m0, p.rank);  // this rank's sequence slice on the owner
        const uint32_t srow = smem_u32(smem_c) + row_in_tile * 128;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          if (issuer) tma_store_wait_read<0>();  // previous stores have finished reading the staging buffer
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + (half * 4 + cc) * 32, r);
            tmem_ld_wait();
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float lo = __uint_as_float(r[2 * i]), hi = __uint_as_float(r[2 * i + 1]);
              if (tl.kblocks == 0) { lo = 0.f; hi = 0.f; }  // empty group: nothing was accumulated
              if (p.is_bf16) {
                pk[i] = pack_bf16x2(lo, hi);
              } else {
                __half2 h = __floats2half2_rn(lo, hi);
                pk[i] = *reinterpret_cast<uint32_t*>(&h);
              }
            }
            const uint32_t box = srow + (cc >> 1) * 16384;  // 64-column box inside the half
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t chunk = (uint32_t)((cc & 1) * 4 + i) ^ (uint32_t)(row_in_tile & 7);  // 128B swizzle
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(box + chunk * 16), "r"(pk[4 * i]),
                           "r"(pk[4 * i + 1]), "r"(pk[4 * i + 2]), "r"(pk[4 * i + 3])
                           : "memory");
            }
          }
          if (half == 1) {  // all TMEM reads of this accumulator are done
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
          }
          fence_proxy_async();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (issuer) {
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              const int x = tl.n0 + half * 128 + b * 64;
              if (x >= p.N) continue;
              if (p.mode == SCATTER_N) {  // the 64-column box goes to the rank that owns those heads
                const int owner = x / p.n_shard;
                tma_store_2d(&cmaps.m[owner], smem_c + b * 16384, x - owner * p.n_shard, y);
              } else {
                tma_store_2d(cm, smem_c + b * 16384, x, y);
              }
            }
            tma_store_commit();
          }
        }
      } else {
        void* cbase = p.C;
        long long ld = p.ldc;
        int out_row = row;
        if (p.mode == GROUPED_K) {
          cbase = p.out_fp32 ? (void*)(reinterpret_cast<float*>(p.C) + (long long)tl.group * p.c_group_stride)
                             : (void*)(reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)tl.group * p.c_group_stride);
        } else if (p.mode == SCATTER) {
          cbase = p.stage_ptrs[dst_rank];
          ld = p.N;
          out_row = p.rank * p.m_shard + (row - dst_rank * p.m_shard);  // slot [src = this rank][local row]
        }
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (tl.kblocks == 0) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          const int col = tl.n0 + c * 32;
          if (row < tl.row_end && col < p.N) store_row32(p, cbase, ld, out_row, col, p.N, r);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }

      if (p.mode == SCATTER) {
        // count finished tiles per owner; whoever completes the last one publishes "my partial is there"
        if (p.tma_store) {
          if (issuer) tma_store_wait_all<0>();  // the bulk stores of this tile are complete
        } else {
          __threadfence_system();
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        if (issuer) {
          __threadfence_system();
          const int tiles_per_owner = (p.m_shard / BM) * ((p.N + BN - 1) / BN);
          const unsigned int done = atomicAdd(p.tile_counters + dst_rank, 1u) + 1u;
          if (done == (unsigned int)tiles_per_owner) {
            p.tile_counters[dst_rank] = 0;  // ready for the next launch
            __threadfence_system();
            st_release_sys(p.peer_flags[dst_rank] + p.rank, p.epoch);
          }
        }
      }
      if (p.mode == SCATTER_N && issuer) {
        // count the delivered 64-column boxes per owner; the last one publishes "this rank's slice is complete"
        tma_store_wait_all<0>();
        __threadfence_system();
        const unsigned int expected = (unsigned int)((p.M / BM) * (p.n_shard / 64));
        const int x_end = min(tl.n0 + BN, p.N);
        for (int x = tl.n0; x < x_end;) {
          const int owner = x / p.n_shard;
          const int stop = min((owner + 1) * p.n_shard, x_end);
          const unsigned int boxes = (unsigned int)((stop - x) / 64);
          const unsigned int done = atomicAdd(p.tile_counters + owner, boxes) + boxes;
          if (done == expected) {
            p.tile_counters[owner] = 0;  // ready for the next launch
            __threadfence_system();
            st_release_sys(p.peer_flags[owner] + p.rank, p.epoch);
          }
          x = stop;
        }
      }
    }
    if (issuer && p.tma_store) tma_store_wait_all<0>();  // nothing in flight when the CTA exits
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

int launch(const AMaps& am, const CUtensorMap& tb_, const CMaps& cm, const GemmParams& p, int grid, cudaStream_t st) {
  TB_CUDA_CHECK(cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  gemm_tcgen05_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(am, tb_, cm, p);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
#endif  // TBG_DEFINE_KERNEL

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n = 148;
  }
  return n;
}

inline CUtensorMapDataType tm_dtype(int dtype) {
  return dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}
inline int make_a_map(CUtensorMap* out, const void* A, int dtype, int a_mn, uint64_t m, uint64_t k, long long lda) {
  if (!a_mn) return tbh::make_tmap_2d(out, A, tm_dtype(dtype), 2, m, k, (uint64_t)lda * 2, BM, BK, 3);
  return tbh::make_tmap_2d(out, A, tm_dtype(dtype), 2, k, m, (uint64_t)lda * 2, 64, 64, 3);
}
inline int make_b_map(CUtensorMap* out, const void* B, int dtype, int b_mn, uint64_t n, uint64_t k, long long ldb) {
  if (!b_mn) return tbh::make_tmap_2d(out, B, tm_dtype(dtype), 2, n, k, (uint64_t)ldb * 2, BN, BK, 3);
  return tbh::make_tmap_2d(out, B, tm_dtype(dtype), 2, k, n, (uint64_t)ldb * 2, 64, 64, 3);
}
// output map: [rows, cols] 16-bit row-major, box {64 cols, 128 rows}, 128B swizzle (matches the staging layout)
inline int make_c_map(CUtensorMap* out, void* C, int dtype, uint64_t rows, uint64_t cols, long long ldc) {
  return tbh::make_tmap_2d(out, C, tm_dtype(dtype), 2, rows, cols, (uint64_t)ldc * 2, BM, 64, 3);
}

}  // namespace tbg
