// MX (microscaling) quantisation for sm_100a: 1x32 blocks, one shared power-of-two scale (e8m0) per block, e4m3 elements.
//
//   block scale exponent  e = ceil(log2(amax / 448))   ("rceil": the block maximum never saturates)   or
//                         e = floor(log2(amax)) - 8    ("floor": the OCP reference; may clip the top of the block)
//   q[i] = e4m3(x[i] * 2^-e),  stored scale byte = e + 127 (amax == 0 -> byte 0 = 2^-127, q = 0)
//
// Two layouts, both reading 16-bit inputs once and writing 1 byte per element + 1 byte per 32 elements:
//   axis = -1 : blocks run along the row (the contraction dim of an [M, K] operand); scales [M, K/32]
//   axis = -2 : blocks run down the rows (32 consecutive rows of one column): the operand that is contracted over its
//               FIRST dim (wgrad: tokens).  q keeps the [R, C] layout; scales [R/32, C].
// `dequantize` writes bf16 back (exact: an e4m3 value times a power of two fits bf16's 8-bit mantissa), which is how the
// quantised operands are fed to the bf16 tensor-core GEMM until the block-scaled MMA path lands.
//
// Semantics: npu_dynamic_mx_quant(axis, dst_type=e4m3, scale_alg) of the reference (patches/torchao_npu/mx_linear.py:
// 38-99, experiments/ao_npu/torchao_npu/ops/mx_ops.py).
#include <cuda_fp8.h>

#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr float E4M3_MAX = 448.f;

__device__ __forceinline__ int block_exponent(float amax, int rceil) {
  if (!(amax > 0.f)) return -127;
  int e;
  if (rceil) {
    // smallest e with amax * 2^-e <= 448
    const float r = amax / E4M3_MAX;
    int ex;
    const float m = frexpf(r, &ex);  // r = m * 2^ex, m in [0.5, 1)
    e = (m == 0.5f) ? ex - 1 : ex;
  } else {
    int ex;
    (void)frexpf(amax, &ex);  // floor(log2(amax)) = ex - 1
    e = (ex - 1) - 8;
  }
  return max(-127, min(127, e));
}

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ float from_e4m3(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// axis -1: one warp handles 32 consecutive blocks of a row per step (lane = block); 4 x 16-byte loads per lane.
template <typename T>
__global__ void __launch_bounds__(256) mx_quant_row_kernel(const T* __restrict__ x, uint8_t* __restrict__ q,
                                                           uint8_t* __restrict__ scales, long long rows, int cols,
                                                           int rceil) {
  const int blocks_per_row = cols / 32;
  const long long total = rows * blocks_per_row;
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < total;
       b += (long long)gridDim.x * blockDim.x) {
    const long long row = b / blocks_per_row;
    const int col0 = (int)(b % blocks_per_row) * 32;
    const T* src = x + row * cols + col0;
    float v[32];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const Vec16<T> t = ld16(src + j * 8);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[j * 8 + i] = to_f(t.v[i]);
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const int e = block_exponent(amax, rceil);
    const float inv = exp2f((float)-e);
    uint32_t packed[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      packed[i] = (uint32_t)to_e4m3(v[4 * i] * inv) | ((uint32_t)to_e4m3(v[4 * i + 1] * inv) << 8) |
                  ((uint32_t)to_e4m3(v[4 * i + 2] * inv) << 16) | ((uint32_t)to_e4m3(v[4 * i + 3] * inv) << 24);
    uint4* dst = reinterpret_cast<uint4*>(q + row * cols + col0);
    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    scales[b] = (uint8_t)(e + 127);
  }
}

// axis -2: a CTA of 256 threads covers a [32 rows x 256 columns] slab; thread = column: coalesced 2-byte reads per row,
// the 32 values of a block sit in one thread.
template <typename T>
__global__ void __launch_bounds__(256) mx_quant_col_kernel(const T* __restrict__ x, uint8_t* __restrict__ q,
                                                           uint8_t* __restrict__ scales, long long rows, int cols,
                                                           int rceil) {
  const int col = blockIdx.x * 256 + threadIdx.x;
  const long long r0 = (long long)blockIdx.y * 32;
  if (col >= cols) return;
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = to_f(x[(r0 + i) * cols + col]);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const int e = block_exponent(amax, rceil);
  const float inv = exp2f((float)-e);
#pragma unroll
  for (int i = 0; i < 32; ++i) q[(r0 + i) * cols + col] = to_e4m3(v[i] * inv);
  scales[(long long)blockIdx.y * cols + col] = (uint8_t)(e + 127);
}

// out[r, c] = e4m3(q[r, c]) * 2^(scale - 127); `col_blocks` selects the scale layout (0: [R, C/32], 1: [R/32, C])
__global__ void __launch_bounds__(256) mx_dequant_kernel(const uint8_t* __restrict__ q,
                                                         const uint8_t* __restrict__ scales,
                                                         __nv_bfloat16* __restrict__ out, long long rows, int cols,
                                                         int col_blocks) {
  const long long n8 = rows * cols / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const long long e0 = i * 8;
    const long long row = e0 / cols;
    const int col = (int)(e0 % cols);
    const uint2 raw = *reinterpret_cast<const uint2*>(q + e0);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
    Vec16<__nv_bfloat16> o;
    if (!col_blocks) {
      const float s = exp2f((float)scales[row * (cols / 32) + col / 32] - 127.f);
#pragma unroll
      for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16(from_e4m3(b[k]) * s);
    } else {
      const uint8_t* sr = scales + (row / 32) * cols + col;
#pragma unroll
      for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16(from_e4m3(b[k]) * exp2f((float)sr[k] - 127.f));
    }
    st16(out + e0, o);
  }
}
// Both layouts from ONE read: a CTA of 256 threads stages a [128 rows x 128 columns] tile in shared memory (8 x 16-byte
// loads in flight per thread), quantises 1x32 blocks along the rows (q1 [R, C], s1 [R, C/32]; two blocks per thread) and
// 32x1 blocks down the rows (one column PAIR per thread, read as packed 2 x 16-bit words), which leave TRANSPOSED
// (q2t [C, R], s2t [C, R/32]): the K-major operand a GEMM contracting over the rows wants (wgrad: tokens; dgrad: the
// weight's output features), with no 16-bit transpose copy in between.  The quantised bytes go back through the same
// shared memory (XOR-swizzled 16-byte chunks) so that both outputs leave as whole 128-byte lines: written straight from
// the registers, every thread's 16-byte pieces landed in a different line and the store path, not DRAM, set the pace
// (28 sectors per request, 2.5x the sectors the data needs).  Block maxima use packed 2 x 16-bit abs / max, the casts
// the paired e4m3x2 conversion.  Either output may be absent (null pointer).
constexpr int DUAL_ROWS = 128, DUAL_COLS = 128, DUAL_STRIDE = DUAL_COLS + 8;  // +16 bytes per row: 16-byte aligned rows
constexpr int DUAL_THREADS = 256;
constexpr int DUAL_Q1_BYTES = DUAL_ROWS * DUAL_COLS;   // staged q1 tile: [row][128 bytes]
constexpr int DUAL_Q2_BYTES = DUAL_COLS * DUAL_ROWS;   // staged q2t tile: [column][128 bytes]
constexpr int DUAL_SMEM = DUAL_ROWS * DUAL_STRIDE * 2; // 34816 bytes: the 16-bit tile; both staged tiles fit inside
static_assert(DUAL_Q1_BYTES + DUAL_Q2_BYTES <= DUAL_SMEM, "staging reuses the input tile");

template <typename T> struct Pair;
template <> struct Pair<__nv_bfloat16> { using type = __nv_bfloat162; };
template <> struct Pair<__half> { using type = __half2; };

__device__ __forceinline__ __nv_bfloat162 absmax2(__nv_bfloat162 m, __nv_bfloat162 v) { return __hmax2(m, __habs2(v)); }
__device__ __forceinline__ __half2 absmax2(__half2 m, __half2 v) { return __hmax2(m, __habs2(v)); }
__device__ __forceinline__ float2 pair_to_f2(__nv_bfloat162 v) { return __bfloat1622float2(v); }
__device__ __forceinline__ float2 pair_to_f2(__half2 v) { return __half22float2(v); }

// two floats -> two e4m3 bytes (a in the low byte)
__device__ __forceinline__ uint32_t to_e4m3x2(float a, float b) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}

template <typename T>
__global__ void __launch_bounds__(DUAL_THREADS) mx_quant_dual_kernel(const T* __restrict__ x, uint8_t* __restrict__ q1,
                                                                     uint8_t* __restrict__ s1,
                                                                     uint8_t* __restrict__ q2t,
                                                                     uint8_t* __restrict__ s2t, long long rows,
                                                                     int cols, int rceil, int atoms) {
  using P2 = typename Pair<T>::type;
  __shared__ __align__(16) uint8_t smem[DUAL_SMEM];
  __shared__ uint32_t s1_stage[DUAL_ROWS], s2_stage[DUAL_COLS];  // 4 scale bytes per tile row / tile column
  T* tile = reinterpret_cast<T*>(smem);
  uint8_t* q1_stage = smem;
  uint8_t* q2_stage = smem + DUAL_Q1_BYTES;
  const int t = threadIdx.x;
  const long long r0 = (long long)blockIdx.x * DUAL_ROWS;
  const int c0 = blockIdx.y * DUAL_COLS;
  {
    Vec16<T> v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int idx = j * DUAL_THREADS + t;
      const int r = idx / 16, c8 = (idx % 16) * 8;
      if (r0 + r < rows && c0 + c8 < cols) {
        v[j] = ld16(x + (r0 + r) * cols + c0 + c8);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[j].v[i] = from_f<T>(0.f);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int idx = j * DUAL_THREADS + t;
      st16(tile + (idx / 16) * DUAL_STRIDE + (idx % 16) * 8, v[j]);
    }
  }
  __syncthreads();

  // ---- quantise into registers (out-of-range blocks of a partial tile quantise the zero fill and are never stored)
  uint32_t rowq[2][8];
  uint8_t rowe[2];
  if (q1 != nullptr) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      // consecutive threads take consecutive rows of one 32-column block: conflict-free 16-byte shared loads
      const int b = k * DUAL_THREADS + t;
      const int r = b % DUAL_ROWS, blk = b / DUAL_ROWS;
      Vec16<T> u[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) u[j] = ld16(tile + r * DUAL_STRIDE + blk * 32 + j * 8);
      const P2* pr = reinterpret_cast<const P2*>(u);  // 16 pairs
      P2 m2 = absmax2(pr[0], pr[0]);
#pragma unroll
      for (int i = 1; i < 16; ++i) m2 = absmax2(m2, pr[i]);
      const float2 mf = pair_to_f2(m2);
      const int e = block_exponent(fmaxf(mf.x, mf.y), rceil);
      const float inv = exp2f((float)-e);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 a = pair_to_f2(pr[2 * i]), c = pair_to_f2(pr[2 * i + 1]);
        rowq[k][i] = to_e4m3x2(a.x * inv, a.y * inv) | (to_e4m3x2(c.x * inv, c.y * inv) << 16);
      }
      rowe[k] = (uint8_t)(e + 127);
    }
  }
  const int cp = t % (DUAL_COLS / 2), rb = t / (DUAL_COLS / 2);  // columns 2cp, 2cp+1; tile rows rb*32 .. +32
  uint32_t pa[8], pb[8];
  uint8_t ea8 = 0, eb8 = 0;
  if (q2t != nullptr) {
    P2 v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = *reinterpret_cast<const P2*>(tile + (rb * 32 + i) * DUAL_STRIDE + 2 * cp);
    P2 m2 = absmax2(v[0], v[0]);
#pragma unroll
    for (int i = 1; i < 32; ++i) m2 = absmax2(m2, v[i]);
    const float2 mf = pair_to_f2(m2);
    const int ea = block_exponent(mf.x, rceil), eb = block_exponent(mf.y, rceil);
    const float ia = exp2f((float)-ea), ib = exp2f((float)-eb);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 f0 = pair_to_f2(v[4 * i]), f1 = pair_to_f2(v[4 * i + 1]);
      const float2 f2 = pair_to_f2(v[4 * i + 2]), f3 = pair_to_f2(v[4 * i + 3]);
      pa[i] = to_e4m3x2(f0.x * ia, f1.x * ia) | (to_e4m3x2(f2.x * ia, f3.x * ia) << 16);
      pb[i] = to_e4m3x2(f0.y * ib, f1.y * ib) | (to_e4m3x2(f2.y * ib, f3.y * ib) << 16);
    }
    ea8 = (uint8_t)(ea + 127);
    eb8 = (uint8_t)(eb + 127);
  }
  __syncthreads();  // every read of the 16-bit tile is done: its memory becomes the staging area

  // ---- stage the bytes: 16-byte chunk `ch` of line `l` sits at chunk (ch ^ key(l)) of that line
  if (q1 != nullptr) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int b = k * DUAL_THREADS + t;
      const int r = b % DUAL_ROWS, blk = b / DUAL_ROWS;
      uint4* line = reinterpret_cast<uint4*>(q1_stage + r * DUAL_COLS);
      line[(2 * blk) ^ (r & 7)] = make_uint4(rowq[k][0], rowq[k][1], rowq[k][2], rowq[k][3]);
      line[(2 * blk + 1) ^ (r & 7)] = make_uint4(rowq[k][4], rowq[k][5], rowq[k][6], rowq[k][7]);
      reinterpret_cast<uint8_t*>(s1_stage + r)[blk] = rowe[k];
    }
  }
  if (q2t != nullptr) {
    uint4* la = reinterpret_cast<uint4*>(q2_stage + (2 * cp) * DUAL_ROWS);
    uint4* lb = reinterpret_cast<uint4*>(q2_stage + (2 * cp + 1) * DUAL_ROWS);
    const int key = cp & 7;  // the same key for both columns of the pair
    la[(2 * rb) ^ key] = make_uint4(pa[0], pa[1], pa[2], pa[3]);
    la[(2 * rb + 1) ^ key] = make_uint4(pa[4], pa[5], pa[6], pa[7]);
    lb[(2 * rb) ^ key] = make_uint4(pb[0], pb[1], pb[2], pb[3]);
    lb[(2 * rb + 1) ^ key] = make_uint4(pb[4], pb[5], pb[6], pb[7]);
    reinterpret_cast<uint8_t*>(s2_stage + 2 * cp)[rb] = ea8;
    reinterpret_cast<uint8_t*>(s2_stage + 2 * cp + 1)[rb] = eb8;
  }
  __syncthreads();

  // ---- whole lines out: 8 consecutive threads write the 128 bytes of one output row
  if (q1 != nullptr) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = j * DUAL_THREADS + t;
      const int r = idx / 8, ch = idx % 8;
      if (r0 + r < rows && c0 + ch * 16 < cols)
        *reinterpret_cast<uint4*>(q1 + (r0 + r) * cols + c0 + ch * 16) =
            reinterpret_cast<const uint4*>(q1_stage + r * DUAL_COLS)[ch ^ (r & 7)];
    }
    if (atoms) {
      // the tile's 128 rows x 4 blocks are exactly one 512-byte scale atom of the block-scaled GEMM:
      // byte (row % 32) * 16 + (row / 32) * 4 + block, atoms stored [row block][column block]
      if (t < DUAL_ROWS) {
        uint8_t* atom = s1 + ((r0 / DUAL_ROWS) * (long long)(cols / DUAL_COLS) + c0 / DUAL_COLS) * 512;
        *reinterpret_cast<uint32_t*>(atom + (t % 32) * 16 + (t / 32) * 4) = s1_stage[t];
      }
    } else if (t < DUAL_ROWS && r0 + t < rows) {
      const int sc = cols / 32;  // scale bytes per row of s1
      uint8_t* dst = s1 + (r0 + t) * sc + c0 / 32;
      if (sc % 4 == 0) {  // c0 / 32 is a multiple of 4: an aligned word (a row of sc % 4 == 0 has whole tiles only)
        *reinterpret_cast<uint32_t*>(dst) = s1_stage[t];
      } else {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(s1_stage + t);
        for (int i = 0; i < 4 && c0 / 32 + i < sc; ++i) dst[i] = src[i];
      }
    }
  }
  if (q2t != nullptr) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = j * DUAL_THREADS + t;
      const int c = idx / 8, ch = idx % 8;
      if (c0 + c < cols && r0 + ch * 16 < rows)
        *reinterpret_cast<uint4*>(q2t + (long long)(c0 + c) * rows + r0 + ch * 16) =
            reinterpret_cast<const uint4*>(q2_stage + c * DUAL_ROWS)[ch ^ ((c >> 1) & 7)];
    }
    if (atoms) {
      if (t >= DUAL_ROWS) {  // the transposed operand's rows are this tile's columns, its blocks this tile's row blocks
        const int c = t - DUAL_ROWS;
        uint8_t* atom = s2t + ((long long)(c0 / DUAL_COLS) * (rows / DUAL_ROWS) + r0 / DUAL_ROWS) * 512;
        *reinterpret_cast<uint32_t*>(atom + (c % 32) * 16 + (c / 32) * 4) = s2_stage[c];
      }
    } else if (t >= DUAL_ROWS && c0 + (t - DUAL_ROWS) < cols) {  // the other half of the CTA takes the column scales
      const int c = t - DUAL_ROWS;
      const long long sr = rows / 32;  // scale bytes per row of s2t
      uint8_t* dst = s2t + (long long)(c0 + c) * sr + r0 / 32;
      if (sr % 4 == 0) {
        *reinterpret_cast<uint32_t*>(dst) = s2_stage[c];
      } else {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(s2_stage + c);
        for (int i = 0; i < 4 && r0 / 32 + i < sr; ++i) dst[i] = src[i];
      }
    }
  }
}
}  // namespace

// x: [rows, cols] bf16 (dtype 1) or fp16 (dtype 2).  axis -1: cols % 32 == 0, scales [rows, cols/32].
// axis -2: rows % 32 == 0, scales [rows/32, cols].  q: [rows, cols] bytes (e4m3).  round: 0 floor, 1 rceil.
TB_API int tb_mx_quantize(const void* x, void* q, void* scales, long long rows, int cols, int axis, int round, int dtype,
                          cudaStream_t st) {
  if (rows == 0 || cols == 0) return 0;
  if ((dtype != 1 && dtype != 2) || (axis != -1 && axis != -2) || cols % 8 != 0) return TB_ERR_ARG;
  if (axis == -1) {
    if (cols % 32 != 0) return TB_ERR_ARG;
    const long long total = rows * (cols / 32);
    const int grid = (int)min((total + 255) / 256, (long long)148 * 16);
    if (dtype == 1)
      mx_quant_row_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, (uint8_t*)scales,
                                                               rows, cols, round);
    else
      mx_quant_row_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, (uint8_t*)q, (uint8_t*)scales, rows, cols,
                                                        round);
  } else {
    if (rows % 32 != 0 || rows / 32 > 65535) return TB_ERR_ARG;
    dim3 grid((cols + 255) / 256, (unsigned)(rows / 32));
    if (dtype == 1)
      mx_quant_col_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, (uint8_t*)scales,
                                                               rows, cols, round);
    else
      mx_quant_col_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, (uint8_t*)q, (uint8_t*)scales, rows, cols,
                                                        round);
  }
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

TB_API int tb_mx_dequantize(const void* q, const void* scales, void* out, long long rows, int cols, int axis,
                            cudaStream_t st) {
  if (rows == 0 || cols == 0) return 0;
  if ((axis != -1 && axis != -2) || cols % 8 != 0 || (axis == -1 && cols % 32 != 0) || (axis == -2 && rows % 32 != 0))
    return TB_ERR_ARG;
  const long long n8 = rows * cols / 8;
  const int grid = (int)min((n8 + 255) / 256, (long long)148 * 16);
  mx_dequant_kernel<<<grid, 256, 0, st>>>((const uint8_t*)q, (const uint8_t*)scales, (__nv_bfloat16*)out, rows, cols,
                                          axis == -2 ? 1 : 0);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

// One pass over x [rows, cols] (bf16 dtype 1 / fp16 dtype 2; rows % 32 == 0, cols % 32 == 0) producing
//   q1 [rows, cols] e4m3 + s1 [rows, cols/32]   (blocks along the row), and / or
//   q2t [cols, rows] e4m3 + s2t [cols, rows/32] (blocks down the rows, written transposed).
// A null q1 or q2t skips that output.  atoms != 0 (rows % 128 == 0 and cols % 128 == 0) writes the scales in the
// 512-byte atom order the block-scaled GEMM reads: s1 as [rows/128][cols/128][512], s2t as [cols/128][rows/128][512].
TB_API int tb_mx_quantize_dual(const void* x, void* q1, void* s1, void* q2t, void* s2t, long long rows, int cols,
                               int round, int dtype, int atoms, cudaStream_t st) {
  if (rows == 0 || cols == 0) return 0;
  if ((dtype != 1 && dtype != 2) || rows % 32 != 0 || cols % 32 != 0) return TB_ERR_ARG;
  if (atoms && (rows % DUAL_ROWS != 0 || cols % DUAL_COLS != 0)) return TB_ERR_ARG;
  if ((q1 == nullptr) != (s1 == nullptr) || (q2t == nullptr) != (s2t == nullptr) || (q1 == nullptr && q2t == nullptr))
    return TB_ERR_ARG;
  const long long row_tiles = (rows + DUAL_ROWS - 1) / DUAL_ROWS;
  const int col_tiles = (cols + DUAL_COLS - 1) / DUAL_COLS;
  if (row_tiles > 0x7fffffffLL || col_tiles > 65535) return TB_ERR_ARG;
  dim3 grid((unsigned)row_tiles, (unsigned)col_tiles);
  if (dtype == 1)
    mx_quant_dual_kernel<__nv_bfloat16><<<grid, DUAL_THREADS, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q1, (uint8_t*)s1,
                                                              (uint8_t*)q2t, (uint8_t*)s2t, rows, cols, round, atoms);
  else
    mx_quant_dual_kernel<__half><<<grid, DUAL_THREADS, 0, st>>>((const __half*)x, (uint8_t*)q1, (uint8_t*)s1, (uint8_t*)q2t,
                                                       (uint8_t*)s2t, rows, cols, round, atoms);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
