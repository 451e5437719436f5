// Backward of the lightning-indexer score  score[s, t] = Σ_h w[s, h] · relu(x[s, h, t])  with x = q_idx · k_idxᵀ:
//
//   dx[s, h, t] = dscore[s, t] · w[s, h] · [x[s, h, t] > 0]          (storage dtype, feeds the two GEMMs of dq / dk)
//   dw[s, h]    = Σ_t dscore[s, t] · relu(x[s, h, t])                 (fp32)
//
// One CTA per (query, head) row of x: the row is read once, dx written once, dscore[s, :] is shared by the heads of a
// query (L2 hits).  In PyTorch the same costs a handful of passes over fp32 [queries, heads, keys] tensors (relu, its
// mask, a broadcast multiply, a reduction), which was the largest item of a DeepSeek-V3.2 step.
//
// Part of what the reference's `npu_sparse_lightning_indexer_grad_kl_loss` (K10) fuses.
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

template <typename T>
__global__ void __launch_bounds__(256) indexer_relu_bwd_kernel(const T* __restrict__ x, const float* __restrict__ dscore,
                                                               const float* __restrict__ w, T* __restrict__ dx,
                                                               float* __restrict__ dw, int heads, int cols) {
  constexpr int V = Vec16<T>::N;
  __shared__ float part[8];
  const long long row = blockIdx.x;  // (s, h)
  const long long s = row / heads;
  const T* xr = x + row * cols;
  T* dr = dx + row * cols;
  const float* g = dscore + s * cols;
  const float wh = w[row];
  float acc = 0.f;
  for (int c = threadIdx.x * V; c < cols; c += 256 * V) {
    const Vec16<T> v = ld16(xr + c);
    Vec16<T> o;
#pragma unroll
    for (int k = 0; k < V; k += 4) {
      const float4 g4 = *reinterpret_cast<const float4*>(g + c + k);
      const float gg[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float xv = to_f(v.v[k + e]);
        const bool pos = xv > 0.f;
        acc = fmaf(gg[e], pos ? xv : 0.f, acc);
        o.v[k + e] = from_f<T>(pos ? gg[e] * wh : 0.f);
      }
    }
    st16(dr + c, o);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += part[i];
    dw[row] = t;
  }
}

}  // namespace

// x, dx: [rows = queries * heads, cols] (dtype 1 bf16 / 2 fp16 / 0 fp32); dscore [queries, cols] fp32; w, dw [rows] fp32.
// cols a multiple of 8 (4 for fp32).
TB_API int tb_indexer_relu_bwd(const void* x, const float* dscore, const float* w, void* dx, float* dw, long long rows,
                               int heads, int cols, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (heads <= 0 || cols <= 0 || rows % heads || rows > 0x7fffffffLL) return TB_ERR_ARG;
  if (cols % (dtype == 0 ? 4 : 8)) return TB_ERR_ARG;
  if (dtype == 0)
    indexer_relu_bwd_kernel<float><<<(unsigned)rows, 256, 0, st>>>((const float*)x, dscore, w, (float*)dx, dw, heads,
                                                                  cols);
  else if (dtype == 1)
    indexer_relu_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>((const __nv_bfloat16*)x, dscore, w,
                                                                          (__nv_bfloat16*)dx, dw, heads, cols);
  else if (dtype == 2)
    indexer_relu_bwd_kernel<__half><<<(unsigned)rows, 256, 0, st>>>((const __half*)x, dscore, w, (__half*)dx, dw,
                                                                   heads, cols);
  else
    return TB_ERR_ARG;
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
