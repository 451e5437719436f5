// Fast Walsh-Hadamard transform over the last dim (n = 64, 128, 256 or 512), bf16 / fp16 in and out, fp32 butterflies.
//
// One warp per row: lane l holds n/32 consecutive elements; the first log2(n/32) butterfly stages stay inside the
// registers of a lane, the last five exchange with xor-shuffles.  The matrix is symmetric and orthogonal up to the
// scale, so the backward pass is the same transform applied to the gradient.
//
// Semantics: rotate_activation(x) = x @ H_n * n^-0.5 of the indexer (reference models/deepseek_v4/model.py:90-112;
// the dense matmul with a materialised Hadamard matrix becomes n log n butterflies).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

template <typename T, int PER>  // PER = n / 32 elements per lane
__global__ void __launch_bounds__(256) hadamard_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows,
                                                       float scale) {
  constexpr int N = PER * 32;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  float v[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) v[i] = to_f(x[row * N + lane * PER + i]);
  // stages inside the lane: element index bits 0 .. log2(PER)-1
#pragma unroll
  for (int h = 1; h < PER; h <<= 1)
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if ((i & h) == 0) {
        const float a = v[i], b = v[i | h];
        v[i] = a + b;
        v[i | h] = a - b;
      }
  // stages across lanes: element index bits log2(PER) .. : lane bits 0..4
#pragma unroll
  for (int m = 1; m < 32; m <<= 1)
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = (lane & m) ? other - v[i] : v[i] + other;
    }
#pragma unroll
  for (int i = 0; i < PER; ++i) y[row * N + lane * PER + i] = from_f<T>(v[i] * scale);
}

template <typename T>
int launch(const void* x, void* y, long long rows, int n, float scale, cudaStream_t st) {
  const unsigned grid = (unsigned)((rows + 7) / 8);
  switch (n) {
    case 64: hadamard_kernel<T, 2><<<grid, 256, 0, st>>>((const T*)x, (T*)y, rows, scale); break;
    case 128: hadamard_kernel<T, 4><<<grid, 256, 0, st>>>((const T*)x, (T*)y, rows, scale); break;
    case 256: hadamard_kernel<T, 8><<<grid, 256, 0, st>>>((const T*)x, (T*)y, rows, scale); break;
    case 512: hadamard_kernel<T, 16><<<grid, 256, 0, st>>>((const T*)x, (T*)y, rows, scale); break;
    default: return TB_ERR_ARG;
  }
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
}  // namespace

// x, y: [rows, n] contiguous (y may alias x); dtype 1 = bf16, 2 = fp16.
TB_API int tb_hadamard(const void* x, void* y, long long rows, int n, float scale, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (dtype == 1) return launch<__nv_bfloat16>(x, y, rows, n, scale, st);
  if (dtype == 2) return launch<__half>(x, y, rows, n, scale, st);
  return TB_ERR_ARG;
}
