// Block-scaled MXFP8 GEMM on the 5th-generation tensor cores:
//
//   C[M,N] (bf16) = Σ_k  (A_q[m,k] · 2^(SA[m,k/32]-127)) · (B_q[n,k] · 2^(SB[n,k/32]-127))
//
// A_q [M,K], B_q [N,K]: e4m3 bytes, K contiguous.  SA / SB: e8m0 bytes, one per 32 elements of K, handed over in
// "atom" order (see below).  The scaling happens INSIDE the MMA (`tcgen05.mma.kind::mxf8f6f4.block_scale`): the
// scale bytes travel global -> shared (bulk copy) -> tensor memory (`tcgen05.cp`) next to the operand tiles, so the
// GEMM reads one byte per element and runs at the fp8 rate.
//
// Roles (192 threads, persistent, one CTA per SM): warp 0 lane 0 = TMA producer, warp 1 lane 0 = MMA issuer (also
// issues the scale copies into tensor memory), warps 2..5 = epilogue (tcgen05.ld -> bf16 -> swizzled staging -> TMA
// store).  Stage = 128 K-elements: A 128x128 B, B XBNx128 B (128B-swizzled), one scale atom of 512 B per 128 rows.
//
// Scale atom: the scales of 128 rows x 4 consecutive K-blocks (= one stage), 512 bytes, byte offset of
// (row = 32*m1 + m0, block kb) is  m0*16 + m1*4 + kb.  `tcgen05.cp.32x128b.warpx4` copies the 32 rows x 16 bytes of an
// atom into 4 tensor-memory columns of every lane quarter; the MMA of K-step kb selects byte kb of each column
// through the scale-factor id fields of its instruction descriptor.  Atoms are stored [row block][stage] in global
// memory so one 512-byte bulk copy fetches one.
//
// Two tile shapes (template parameter XBN): 128x256 with ONE accumulator (the next tile's MMAs wait for the epilogue to
// drain it; least operand traffic per flop) and 128x128 with TWO accumulators and six stages (the epilogue of a tile
// overlaps the MMAs of the next).  Tensor memory: columns 0..255 accumulators, 256.. scale slots (16 columns per
// stage: 4 for A, up to 8 for B).
//
// Every wait is bounded (gemm_core.cuh `wait_bounded`); on expiry: status word, CTA abort flag, drain, free TMEM.
//
// Reference counterpart: the MXFP8 linear / grouped GEMM of torchtitan_npu/converters/lowp (mx_linear.py:26-100,
// mxfp8_grouped_mm.py:22-109), which call `npu_quant_matmul` / `npu_grouped_matmul` with e8m0 block scales.
#include "../gemm/gemm_core.cuh"

using namespace tbg;

namespace {

constexpr int XBK = 128;                       // K elements (= bytes) per stage
constexpr int XA_STAGE = BM * XBK;             // 16 KB
constexpr int SF_ATOM = 512;
constexpr int XC_STAGE = 16 * 1024;            // epilogue staging: one 128 x 64 bf16 box
constexpr int SF_TMEM_BASE = 256;              // first scale column
constexpr int SF_TMEM_PER_STAGE = 16;

template <int XBN>
struct Cfg {
  static constexpr int STAGES = XBN == 128 ? 6 : 4;
  static constexpr int NACC = XBN == 128 ? 2 : 1;
  static constexpr int B_STAGE = XBN * XBK;
  static constexpr int B_ATOMS = XBN / 128;
  static constexpr int SF_STAGE = (1 + B_ATOMS) * SF_ATOM;
  static constexpr int SMEM = STAGES * (XA_STAGE + B_STAGE + SF_STAGE) + XC_STAGE + 1024 + 256;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
  static_assert(SF_TMEM_BASE + STAGES * SF_TMEM_PER_STAGE <= TMEM_COLS && NACC * XBN <= SF_TMEM_BASE, "TMEM budget");
};

// Grouped forms (rows of the token operand sorted by expert, every group a multiple of 128 rows, `offs` = cumulative
// group ends on the device):
//   GROUP_B_ROWS   C[T, N]   = A[T, K] . B[e]^T     B stacked by rows [E*N, K]: the tile's expert picks its B rows
//   GROUP_B_SLICE  C[T, N]   = A[T, K] . B_e^T      B [N, E*K]: the expert picks a K-slice of B (a weight quantised
//                                                   along its output features and transposed in one pass)
//   GROUP_K        C[e][M,N] = A[M, T_e] . B[N, T_e]^T   the contraction runs over the expert's own token range
// A tile whose contraction range is empty (rows past the last group; an expert without tokens) is written as zeros.
enum XMode : int { X_PLAIN = 0, X_GROUP_B_ROWS = 1, X_GROUP_K = 2, X_GROUP_B_SLICE = 3 };

struct XParams {
  int M, N, K;
  const uint8_t* sfa;  // [M/128][K/128][512]
  const uint8_t* sfb;  // [B rows/128][B stages][512]
  int* status;
  int mode, groups;
  const int* offs;     // [groups] cumulative row ends (multiples of 128)
};

struct XTile {
  int m0, n0;      // tile origin inside one problem
  int b_row;       // first B row of the tile
  int b_ks;        // stage offset of B along its contraction dim
  int c_row;       // first output row
  int ks0, ks1;    // contraction stages [ks0, ks1)
};

// first group whose end lies above `row`, or `groups` when there is none
__device__ __forceinline__ int group_of_row(const int* __restrict__ offs, int groups, int row) {
  int lo = 0, hi = groups;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(offs + mid) > row) hi = mid; else lo = mid + 1;
  }
  return lo;
}

// instruction descriptor of kind::mxf8f6f4 with block scaling: [4,6) B scale id | [7,10) A format (0 = e4m3) |
// [10,13) B format | 15/16 A/B major (0 = K) | [17,23) N >> 3 | 23 scale format (1 = ue8m0) | [24,29) M >> 4 |
// [29,31) A scale id
__device__ __forceinline__ uint32_t idesc_mxf8(int m, int n, uint32_t sf_id) {
  return (sf_id << 4) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(m >> 4) << 24) | (sf_id << 29);
}

__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t sfa,
                                          uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}

// The same instruction with the two descriptors given as (low, high) words: the issuing thread keeps the layout
// halves in registers and only adds stage / k offsets to the start-address field.
__device__ __forceinline__ void umma_mxf8_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "mov.b64 da, {%1, %2};\n"
      "mov.b64 db, {%3, %4};\n"
      "setp.ne.b32 p, %8, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, %5, [%6], [%7], p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}

// 32 rows x 16 bytes of shared memory -> 4 columns of tensor memory, replicated into the four lane quarters
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint32_t smem_addr) {
  const uint64_t desc = make_smem_desc(smem_addr, 16, 128, 0);  // no swizzle; 8-row groups 128 B apart
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void tmem_cp_sf_lohi(uint32_t taddr, uint32_t lo, uint32_t hi) {
  asm volatile(
      "{\n"
      ".reg .b64 d;\n"
      "mov.b64 d, {%1, %2};\n"
      "tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n"
      "}\n" ::"r"(taddr), "r"(lo), "r"(hi)
      : "memory");
}

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int XBN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
mxfp8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ XParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using C = Cfg<XBN>;
  constexpr int XSTAGES = C::STAGES, XB_STAGE = C::B_STAGE, XSF_STAGE = C::SF_STAGE, NACC = C::NACC;
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem_a + XSTAGES * XA_STAGE;
  uint8_t* smem_c = smem_b + XSTAGES * XB_STAGE;  // 16 KB staging, 1024-byte aligned
  uint8_t* smem_sf = smem_c + XC_STAGE;           // [XSTAGES][1 + B_ATOMS][512]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_sf + XSTAGES * XSF_STAGE);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + XSTAGES;
  uint64_t* tmem_full_bar = bars + 2 * XSTAGES;   // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;   // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < XSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full_bar[a], 1); mbar_init(&tmem_empty_bar[a], 4); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
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
  const int num_m = p.M / BM, num_n = (p.N + XBN - 1) / XBN, kstages = p.K / XBK;
  const int tiles_per_problem = num_m * num_n;
  const int num_tiles = p.mode == X_GROUP_K ? tiles_per_problem * p.groups : tiles_per_problem;
  const int b_stages = p.mode == X_GROUP_B_SLICE ? kstages * p.groups : kstages;  // scale atoms per B row block

  auto tile_of = [&](int t) {  // grouped raster: GROUP_M row tiles share their B columns in L2
    XTile ti;
    const int problem = t / tiles_per_problem;
    t -= problem * tiles_per_problem;
    const int per_group = GROUP_M * num_n;
    const int group = t / per_group, first_m = group * GROUP_M;
    const int gsize = min(num_m - first_m, GROUP_M);
    const int in_group = t - group * per_group;
    ti.m0 = (first_m + in_group % gsize) * BM;
    ti.n0 = (in_group / gsize) * XBN;
    ti.b_row = ti.n0; ti.b_ks = 0; ti.c_row = ti.m0; ti.ks0 = 0; ti.ks1 = kstages;
    if (p.mode == X_GROUP_B_ROWS || p.mode == X_GROUP_B_SLICE) {
      const int e = group_of_row(p.offs, p.groups, ti.m0);
      if (e >= p.groups) ti.ks1 = 0;  // padding rows past the last group
      else if (p.mode == X_GROUP_B_ROWS) ti.b_row = e * p.N + ti.n0;
      else ti.b_ks = e * kstages;
    } else if (p.mode == X_GROUP_K) {
      const int begin = problem == 0 ? 0 : __ldg(p.offs + problem - 1);
      const int end = __ldg(p.offs + problem);
      ti.ks0 = min(max(begin / XBK, 0), kstages);
      ti.ks1 = min(max(end / XBK, ti.ks0), kstages);
      ti.c_row = problem * p.M + ti.m0;
    }
    return ti;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const XTile ti = tile_of(t);
        const int m0 = ti.m0, n0 = ti.n0;
        const bool second_b = C::B_ATOMS == 2 && n0 + 128 < p.N;  // the tile's upper 128 columns exist
        for (int ks = ti.ks0; ks < ti.ks1; ++ks) {
          if (!wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag)) {
            if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_EMPTY); }
            ok = false; break;
          }
          mbar_expect_tx(&full_bar[stage], XA_STAGE + XB_STAGE + (second_b ? 3 : 2) * SF_ATOM);
          tma_load_2d(smem_a + stage * XA_STAGE, &tmap_a, &full_bar[stage], ks * XBK, m0);
          tma_load_2d(smem_b + stage * XB_STAGE, &tmap_b, &full_bar[stage], (ks + ti.b_ks) * XBK, ti.b_row);
          uint8_t* sf = smem_sf + stage * XSF_STAGE;
          bulk_g2s(sf, p.sfa + ((long long)(m0 / 128) * kstages + ks) * SF_ATOM, SF_ATOM, &full_bar[stage]);
          const uint8_t* sfb0 = p.sfb + ((long long)(ti.b_row / 128) * b_stages + ks + ti.b_ks) * SF_ATOM;
          bulk_g2s(sf + SF_ATOM, sfb0, SF_ATOM, &full_bar[stage]);
          if (second_b) bulk_g2s(sf + 2 * SF_ATOM, sfb0 + (long long)b_stages * SF_ATOM, SF_ATOM, &full_bar[stage]);
          if (++stage == XSTAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      int acc = 0; uint32_t acc_phase = 0;
      // Descriptors of stage 0: K-major, 128-byte swizzled rows (128 fp8 each), 8-row atoms 1024 B apart; a K step of
      // 32 elements = +32 B.  The loop adds stage / k offsets to the start-address words only.
      const uint64_t da0 = make_smem_desc(smem_u32(smem_a), 16, 1024, 2);
      const uint64_t db0 = make_smem_desc(smem_u32(smem_b), 16, 1024, 2);
      const uint64_t ds0 = make_smem_desc(smem_u32(smem_sf), 16, 128, 0);  // scale atoms: no swizzle, 8-row groups 128 B apart
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32), s_hi = (uint32_t)(ds0 >> 32);
      const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0, s_lo0 = (uint32_t)ds0;
      const uint32_t id0 = idesc_mxf8(BM, XBN, 0), id1 = idesc_mxf8(BM, XBN, 1), id2 = idesc_mxf8(BM, XBN, 2),
                     id3 = idesc_mxf8(BM, XBN, 3);
      static_assert(XBK / 32 == 4, "four scale blocks per stage");
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const XTile ti = tile_of(t);
        if (ti.ks0 >= ti.ks1) continue;  // nothing to contract: the epilogue writes zeros without an accumulator
        if (!wait_bounded(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag)) {
          if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMEM_EMPTY); }
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * XBN;
        uint32_t accum = 0;  // the first MMA of a tile overwrites the accumulator
        for (int ks = ti.ks0; ks < ti.ks1; ++ks) {
          if (!wait_bounded(&full_bar[stage], phase, abort_flag)) {
            if (*abort_flag == 0) { *abort_flag = 1; if (p.status) atomicExch(p.status, TB_ERR_WAIT_TMA); }
            ok = false; break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + (uint32_t)stage * (XA_STAGE >> 4);
          const uint32_t b_lo = b_lo0 + (uint32_t)stage * (XB_STAGE >> 4);
          const uint32_t s_lo = s_lo0 + (uint32_t)stage * (XSF_STAGE >> 4);
          const uint32_t sfa_t = tmem_base + SF_TMEM_BASE + stage * SF_TMEM_PER_STAGE;
          const uint32_t sfb_t = sfa_t + 4;
          tmem_cp_sf_lohi(sfa_t, s_lo, s_hi);
          tmem_cp_sf_lohi(sfb_t, s_lo + (SF_ATOM >> 4), s_hi);
          if (C::B_ATOMS == 2) tmem_cp_sf_lohi(sfb_t + 4, s_lo + 2 * (SF_ATOM >> 4), s_hi);
          umma_mxf8_lohi(d_tmem, a_lo, a_hi, b_lo, b_hi, id0, sfa_t, sfb_t, accum);
          umma_mxf8_lohi(d_tmem, a_lo + 2, a_hi, b_lo + 2, b_hi, id1, sfa_t, sfb_t, 1u);
          umma_mxf8_lohi(d_tmem, a_lo + 4, a_hi, b_lo + 4, b_hi, id2, sfa_t, sfb_t, 1u);
          umma_mxf8_lohi(d_tmem, a_lo + 6, a_hi, b_lo + 6, b_hi, id3, sfa_t, sfb_t, 1u);
          accum = 1u;
          umma_commit(&empty_bar[stage]);
          if (++stage == XSTAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full_bar[acc]);
        if (++acc == NACC) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int q = warp & 3;
    const bool issuer = warp == 2 && lane == 0;
    int acc = 0; uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const XTile ti = tile_of(t);
      const int n0 = ti.n0;
      const bool zero_tile = ti.ks0 >= ti.ks1;  // uniform over the four epilogue warps
      bool ok = zero_tile || wait_bounded(&tmem_full_bar[acc], acc_phase, abort_flag);
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
      const int row_in_tile = q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * XBN + ((uint32_t)(q * 32) << 16);
      const uint32_t srow = smem_u32(smem_c) + row_in_tile * 128;
#pragma unroll 1
      for (int box = 0; box < XBN / 64; ++box) {  // 64-column boxes through one staging buffer
        if (issuer) tma_store_wait_read<0>();  // the previous store has finished reading the buffer
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t pk[16];
          if (zero_tile) {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = 0u;
          } else {
            uint32_t r[32];
            tmem_ld_32x32(taddr + (box * 2 + cc) * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t chunk = (uint32_t)(cc * 4 + i) ^ (uint32_t)(row_in_tile & 7);  // 128B swizzle
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + chunk * 16), "r"(pk[4 * i]),
                         "r"(pk[4 * i + 1]), "r"(pk[4 * i + 2]), "r"(pk[4 * i + 3])
                         : "memory");
          }
        }
        if (!zero_tile && box == XBN / 64 - 1) {  // all reads of the accumulator are done
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
        }
        fence_proxy_async();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (issuer) {
          const int x = n0 + box * 64;
          if (x < p.N) tma_store_2d(&tmap_c, smem_c, x, ti.c_row);
          tma_store_commit();
        }
      }
      if (!zero_tile && ++acc == NACC) { acc = 0; acc_phase ^= 1; }
    }
    if (issuer) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

int sm_count_x() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n = 148;
  }
  return n;
}

template <int XBN>
int launch_x(const void* A, const void* B, void* C, const XParams& p, cudaStream_t st) {
  CUtensorMap ta, tb_, tc;
  if (int rc = tbh::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)p.K,
                                 BM, XBK, 3))
    return rc;
  const uint64_t g = p.mode == X_PLAIN ? 1 : (uint64_t)p.groups;
  const uint64_t b_rows = p.mode == X_GROUP_B_ROWS ? g * p.N : (uint64_t)p.N;
  const uint64_t b_cols = p.mode == X_GROUP_B_SLICE ? g * p.K : (uint64_t)p.K;
  const uint64_t c_rows = p.mode == X_GROUP_K ? g * p.M : (uint64_t)p.M;
  if (int rc = tbh::make_tmap_2d(&tb_, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_rows, b_cols, b_cols, XBN, XBK, 3))
    return rc;
  if (int rc = tbh::make_tmap_2d(&tc, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c_rows, (uint64_t)p.N,
                                 (uint64_t)p.N * 2, BM, 64, 3))
    return rc;
  const long long tiles_ll = (long long)(p.M / BM) * ((p.N + XBN - 1) / XBN) * (p.mode == X_GROUP_K ? p.groups : 1);
  if (tiles_ll > 0x7fffffffLL) return TB_ERR_ARG;
  const int tiles = (int)tiles_ll;
  const int grid = tiles < sm_count_x() ? tiles : sm_count_x();
  TB_CUDA_CHECK(cudaFuncSetAttribute(mxfp8_gemm_kernel<XBN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg<XBN>::SMEM));
  mxfp8_gemm_kernel<XBN><<<grid, NUM_THREADS, Cfg<XBN>::SMEM, st>>>(ta, tb_, tc, p);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

}  // namespace

// A_q [M,K], B_q [N,K] e4m3 (K contiguous); sfa [M/128][K/128][512], sfb [ceil(N/128)][K/128][512] e8m0 atoms;
// C [M,N] bf16.  M % 128 == 0, N % 8 == 0, K % 128 == 0.  tile_n: 128, 256, or 0 = the library's choice.
TB_API int tb_mxfp8_gemm(const void* A, const void* B, const void* sfa, const void* sfb, void* C, int M, int N, int K,
                         int tile_n, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0 || M % BM || N % 8 || K % XBK) return TB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15)) return TB_ERR_ARG;
  if (tile_n != 0 && tile_n != 128 && tile_n != 256) return TB_ERR_ARG;
  XParams p{M, N, K, reinterpret_cast<const uint8_t*>(sfa), reinterpret_cast<const uint8_t*>(sfb), status, X_PLAIN, 1,
            nullptr};
  if (tile_n == 0) tile_n = 256;
  return tile_n == 128 ? launch_x<128>(A, B, C, p, st) : launch_x<256>(A, B, C, p, st);
}

// Grouped block-scaled GEMMs over expert-sorted rows whose groups are multiples of 128 rows.  `offs` [groups] int32 on
// the device: cumulative group ends.  M, N, K describe ONE problem; the operands are
//   mode 1: A [M = all rows, K], B [groups*N, K] (N % 128 == 0),  C [M, N]
//   mode 3: A [M = all rows, K], B [N, groups*K],                 C [M, N]
//   mode 2: A [M, K = all rows], B [N, K],                        C [groups*M, N]   (contraction over each group's rows)
// with scale atoms laid out like the operands: [rows/128][contraction stages][512].
TB_API int tb_mxfp8_grouped_gemm(const void* A, const void* B, const void* sfa, const void* sfb, void* C, int M, int N,
                                 int K, const int* offs, int groups, int mode, int tile_n, int* status,
                                 cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0 || M % BM || N % 8 || K % XBK || groups <= 0 || offs == nullptr) return TB_ERR_ARG;
  if (mode != X_GROUP_B_ROWS && mode != X_GROUP_K && mode != X_GROUP_B_SLICE) return TB_ERR_ARG;
  if (mode == X_GROUP_B_ROWS && N % 128) return TB_ERR_ARG;  // every expert's scale atoms start on a row block
  if ((reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15)) return TB_ERR_ARG;
  if (tile_n != 0 && tile_n != 128 && tile_n != 256) return TB_ERR_ARG;
  XParams p{M, N, K, reinterpret_cast<const uint8_t*>(sfa), reinterpret_cast<const uint8_t*>(sfb), status, mode, groups,
            offs};
  if (tile_n == 0) tile_n = 256;
  return tile_n == 128 ? launch_x<128>(A, B, C, p, st) : launch_x<256>(A, B, C, p, st);
}
