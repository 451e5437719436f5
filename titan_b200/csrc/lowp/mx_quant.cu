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
// Both layouts from ONE read: a CTA stages a [64 rows x 128 columns] tile in shared memory, then every thread quantises
// one 1x32 block along the row (q1 [R, C], s1 [R, C/32]) and one 32x1 block down the rows, which it writes TRANSPOSED
// (q2t [C, R], s2t [C, R/32]): the K-major operand a GEMM contracting over the rows wants (wgrad: tokens; dgrad: the
// weight's output features), with no bf16 transpose copy in between.  Either output may be absent (null pointer).
constexpr int DUAL_ROWS = 64, DUAL_COLS = 128, DUAL_STRIDE = DUAL_COLS + 8;  // +16 bytes per row: 16-byte aligned rows

template <typename T>
__global__ void __launch_bounds__(256) mx_quant_dual_kernel(const T* __restrict__ x, uint8_t* __restrict__ q1,
                                                            uint8_t* __restrict__ s1, uint8_t* __restrict__ q2t,
                                                            uint8_t* __restrict__ s2t, long long rows, int cols,
                                                            int rceil) {
  __shared__ __align__(16) T tile[DUAL_ROWS * DUAL_STRIDE];
  const int t = threadIdx.x;
  const long long r0 = (long long)blockIdx.x * DUAL_ROWS;
  const int c0 = blockIdx.y * DUAL_COLS;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int idx = j * 256 + t;
    const int r = idx / 16, c8 = (idx % 16) * 8;
    Vec16<T> v;
    if (r0 + r < rows && c0 + c8 < cols) {
      v = ld16(x + (r0 + r) * cols + c0 + c8);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v.v[i] = from_f<T>(0.f);
    }
    st16(tile + r * DUAL_STRIDE + c8, v);
  }
  __syncthreads();
  if (q1 != nullptr) {
    const int r = t / 4, blk = t % 4;
    if (r0 + r < rows && c0 + blk * 32 < cols) {
      float v[32];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const Vec16<T> u = ld16(tile + r * DUAL_STRIDE + blk * 32 + j * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[j * 8 + i] = to_f(u.v[i]);
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
      uint4* dst = reinterpret_cast<uint4*>(q1 + (r0 + r) * cols + c0 + blk * 32);
      dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      s1[(r0 + r) * (cols / 32) + c0 / 32 + blk] = (uint8_t)(e + 127);
    }
  }
  if (q2t != nullptr) {
    const int c = t % DUAL_COLS, rb = t / DUAL_COLS;
    if (c0 + c < cols && r0 + rb * 32 < rows) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = to_f(tile[(rb * 32 + i) * DUAL_STRIDE + c]);
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
      // rows % 32 == 0 and r0 + rb * 32 is a multiple of 32: the 32-byte run is 16-byte aligned
      uint4* dst = reinterpret_cast<uint4*>(q2t + (long long)(c0 + c) * rows + r0 + rb * 32);
      dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      s2t[(long long)(c0 + c) * (rows / 32) + r0 / 32 + rb] = (uint8_t)(e + 127);
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
// A null q1 or q2t skips that output.
TB_API int tb_mx_quantize_dual(const void* x, void* q1, void* s1, void* q2t, void* s2t, long long rows, int cols,
                               int round, int dtype, cudaStream_t st) {
  if (rows == 0 || cols == 0) return 0;
  if ((dtype != 1 && dtype != 2) || rows % 32 != 0 || cols % 32 != 0) return TB_ERR_ARG;
  if ((q1 == nullptr) != (s1 == nullptr) || (q2t == nullptr) != (s2t == nullptr) || (q1 == nullptr && q2t == nullptr))
    return TB_ERR_ARG;
  const long long row_tiles = (rows + DUAL_ROWS - 1) / DUAL_ROWS;
  const int col_tiles = (cols + DUAL_COLS - 1) / DUAL_COLS;
  if (row_tiles > 0x7fffffffLL || col_tiles > 65535) return TB_ERR_ARG;
  dim3 grid((unsigned)row_tiles, (unsigned)col_tiles);
  if (dtype == 1)
    mx_quant_dual_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q1, (uint8_t*)s1,
                                                              (uint8_t*)q2t, (uint8_t*)s2t, rows, cols, round);
  else
    mx_quant_dual_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, (uint8_t*)q1, (uint8_t*)s1, (uint8_t*)q2t,
                                                       (uint8_t*)s2t, rows, cols, round);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
