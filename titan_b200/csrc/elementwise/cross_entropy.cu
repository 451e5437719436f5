// Softmax cross-entropy over large vocabularies for sm_100a.
//
// forward : per row  lse = log Σ exp(x),  loss = lse - x[label]   (0 for ignored rows); one CTA per row,
//           single streaming pass with an online (max, sum) pair in fp32.
// backward: dlogits = (exp(x - lse) - onehot(label)) * gscale[0]   (0 for ignored rows); may write in
//           place over the logits.  `gscale` is a device scalar (upstream gradient of the summed loss).
//
// The logits are read once in forward and once in backward; no fp32 copy of the [T, V] matrix and no
// probability matrix is ever materialised (for T = 8192, V = 128256 that is 4.2 GB per avoided copy).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int CE_THREADS = 512;

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float nm = fmaxf(m, m2);
  if (nm == -INFINITY) { m = nm; s = 0.f; return; }
  s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  m = nm;
}

template <typename T>
__global__ void __launch_bounds__(CE_THREADS) ce_fwd_kernel(const T* __restrict__ logits,
                                                            const long long* __restrict__ labels,
                                                            float* __restrict__ loss, float* __restrict__ lse_out,
                                                            int V, long long pitch, long long ignore_index,
                                                            int* __restrict__ status) {
  constexpr int VEC = Vec16<T>::N;
  const long long row = blockIdx.x;
  const T* x = logits + row * pitch;
  float m = -INFINITY, s = 0.f;
  const int vec_end = (V / VEC) * VEC;
  for (int c = threadIdx.x * VEC; c < vec_end; c += CE_THREADS * VEC) {
    Vec16<T> xv = ld16(x + c);
    float lm = -INFINITY;
#pragma unroll
    for (int i = 0; i < VEC; ++i) lm = fmaxf(lm, to_f(xv.v[i]));
    float ls = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) ls += __expf(to_f(xv.v[i]) - lm);
    online_merge(m, s, lm, ls);
  }
  for (int c = vec_end + threadIdx.x; c < V; c += CE_THREADS) online_merge(m, s, to_f(x[c]), 1.f);
  // warp then block reduction of (m, s)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  __shared__ float sm[CE_THREADS / 32], ss[CE_THREADS / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sm[warp] = m; ss[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    m = lane < CE_THREADS / 32 ? sm[lane] : -INFINITY;
    s = lane < CE_THREADS / 32 ? ss[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_merge(m, s, m2, s2);
    }
    if (lane == 0) {
      const float lse = m + __logf(s);
      lse_out[row] = lse;
      const long long lab = labels[row];
      float l = 0.f;
      if (lab != ignore_index) {
        if (lab < 0 || lab >= V) {
          if (status != nullptr) atomicExch(status, TB_ERR_BOUNDS);
        } else {
          l = lse - to_f(x[lab]);
        }
      }
      loss[row] = l;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(CE_THREADS) ce_bwd_kernel(const T* __restrict__ logits,
                                                            const long long* __restrict__ labels,
                                                            const float* __restrict__ lse,
                                                            const float* __restrict__ gscale, T* __restrict__ dlogits,
                                                            int V, long long pitch, long long ignore_index) {
  constexpr int VEC = Vec16<T>::N;
  const long long row = blockIdx.x;
  const T* x = logits + row * pitch;
  T* d = dlogits + row * pitch;
  const long long lab = labels[row];
  const bool ignored = (lab == ignore_index) || lab < 0 || lab >= V;
  const float g = ignored ? 0.f : gscale[0];
  const float l = lse[row];
  const int vec_end = (V / VEC) * VEC;
  for (int c = threadIdx.x * VEC; c < vec_end; c += CE_THREADS * VEC) {
    Vec16<T> xv = ld16(x + c);
    Vec16<T> o;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float p = __expf(to_f(xv.v[i]) - l);
      if (c + i == lab) p -= 1.f;
      o.v[i] = from_f<T>(p * g);
    }
    st16(d + c, o);
  }
  for (int c = vec_end + threadIdx.x; c < V; c += CE_THREADS) {
    float p = __expf(to_f(x[c]) - l);
    if (c == lab) p -= 1.f;
    d[c] = from_f<T>(p * g);
  }
}
}  // namespace

// dtype: 0 fp32, 1 bf16, 2 fp16.  `pitch` = elements between rows (>= V, multiple of the 16-byte vector).
TB_API int tb_cross_entropy_fwd(const void* logits, const long long* labels, float* loss, float* lse, long long rows,
                                int V, long long pitch, long long ignore_index, int dtype, int* status,
                                cudaStream_t st) {
  if (rows == 0) return 0;
  if (rows > 0x7fffffffLL) return TB_ERR_ARG;
#define TB_CE_F(T)                                                                                              \
  do {                                                                                                          \
    if (pitch % Vec16<T>::N != 0 || (reinterpret_cast<uintptr_t>(logits) & 15) != 0) return TB_ERR_ARG;         \
    ce_fwd_kernel<T><<<(int)rows, CE_THREADS, 0, st>>>((const T*)logits, labels, loss, lse, V, pitch, ignore_index, \
                                                       status);                                                 \
  } while (0)
  switch (dtype) {
    case 0: TB_CE_F(float); break;
    case 1: TB_CE_F(__nv_bfloat16); break;
    case 2: TB_CE_F(__half); break;
    default: return TB_ERR_ARG;
  }
#undef TB_CE_F
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

TB_API int tb_cross_entropy_bwd(const void* logits, const long long* labels, const float* lse, const float* gscale,
                                void* dlogits, long long rows, int V, long long pitch, long long ignore_index,
                                int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  if (rows > 0x7fffffffLL) return TB_ERR_ARG;
#define TB_CE_B(T)                                                                                           \
  do {                                                                                                       \
    if (pitch % Vec16<T>::N != 0 || ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(dlogits)) & 15) != 0) \
      return TB_ERR_ARG;                                                                                     \
    ce_bwd_kernel<T><<<(int)rows, CE_THREADS, 0, st>>>((const T*)logits, labels, lse, gscale, (T*)dlogits, V, pitch, \
                                                       ignore_index);                                        \
  } while (0)
  switch (dtype) {
    case 0: TB_CE_B(float); break;
    case 1: TB_CE_B(__nv_bfloat16); break;
    case 2: TB_CE_B(__half); break;
    default: return TB_ERR_ARG;
  }
#undef TB_CE_B
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
