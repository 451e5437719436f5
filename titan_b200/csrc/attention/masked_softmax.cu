// Row softmax under a selection mask, forward and backward, for the dense form of sparse attention (every key of a
// short key stream goes through one GEMM and the top-k selection becomes a mask).  PyTorch needs about ten elementwise
// passes over the fp32 [heads, queries, keys] logits for this (cast, masked_fill with a broadcast mask, softmax, casts
// back, and their backward); here the logits are read once and the probabilities written once, in the storage dtype.
//
//   P[r, t] = allowed[r % mask_rows, t] ? exp(scale * S[r, t] - m_r) / l_r : 0          (fp32 statistics)
//   dS[r, t] = scale * P[r, t] * (dP[r, t] - Σ_t' P[r, t'] dP[r, t'])
//
// One CTA of 256 threads per row, the row held in registers (up to 64 values per thread: T <= 16384; wider rows take
// two passes over global memory), 16-byte accesses; a row without any allowed key yields zeros.  Rows are [heads * queries]; the mask has one row per query
// and is shared by the heads (row r uses mask row r % mask_rows).
//
// Stands where the reference's sparse attention kernels (`npu_sparse_flash_attention`, K9) apply the top-k selection
// inside their softmax.
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int MS_THREADS = 256;
constexpr int MS_MAX_VECS = 8;  // 16-byte vectors per thread: 8 x 8 bf16 x 256 threads = 16384 columns

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* scratch) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
#pragma unroll
  for (int i = 1; i < MS_THREADS / 32; ++i) r = is_max ? fmaxf(r, scratch[i]) : r + scratch[i];
  return r;
}

template <typename T, int NV>
__global__ void __launch_bounds__(MS_THREADS) masked_softmax_fwd_kernel(const T* __restrict__ S,
                                                                        const unsigned char* __restrict__ allowed,
                                                                        T* __restrict__ P, int cols, int mask_rows,
                                                                        float scale, const float* __restrict__ sink) {
  constexpr int V = Vec16<T>::N;
  __shared__ float scratch[MS_THREADS / 32];
  const long long row = blockIdx.x;
  const T* s = S + row * cols;
  T* p = P + row * cols;
  const unsigned char* a = allowed + (row % mask_rows) * (long long)cols;
  const float sk = sink != nullptr ? sink[row / mask_rows] : -INFINITY;  // per-head logit without a key
  float x[NV][V];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * MS_THREADS + threadIdx.x) * V;
    if (c < cols) {
      const Vec16<T> v = ld16(s + c);
      unsigned char m[V];
      if (V == 8) *reinterpret_cast<uint2*>(m) = *reinterpret_cast<const uint2*>(a + c);
      else *reinterpret_cast<uint32_t*>(m) = *reinterpret_cast<const uint32_t*>(a + c);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        x[i][k] = m[k] ? to_f(v.v[k]) * scale : -INFINITY;
        mx = fmaxf(mx, x[i][k]);
      }
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) x[i][k] = -INFINITY;
    }
  }
  mx = fmaxf(block_reduce(mx, true, scratch), sk);
  const bool empty = mx == -INFINITY;
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int k = 0; k < V; ++k) {
      x[i][k] = empty ? 0.f : __expf(x[i][k] - mx);  // exp(-inf) = 0 for masked columns
      sum += x[i][k];
    }
  sum = block_reduce(sum, false, scratch) + (empty ? 0.f : __expf(sk - mx));  // the sink only feeds the denominator
  const float inv = empty ? 0.f : 1.f / sum;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * MS_THREADS + threadIdx.x) * V;
    if (c < cols) {
      Vec16<T> o;
#pragma unroll
      for (int k = 0; k < V; ++k) o.v[k] = from_f<T>(x[i][k] * inv);
      st16(p + c, o);
    }
  }
}

template <typename T, int NV>
__global__ void __launch_bounds__(MS_THREADS) masked_softmax_bwd_kernel(const T* __restrict__ P,
                                                                        const T* __restrict__ dP,
                                                                        T* __restrict__ dS, int cols, float scale,
                                                                        float* __restrict__ dsink_rows) {
  constexpr int V = Vec16<T>::N;
  __shared__ float scratch[MS_THREADS / 32];
  const long long row = blockIdx.x;
  const T* p = P + row * cols;
  const T* g = dP + row * cols;
  T* d = dS + row * cols;
  float pv[NV][V], gv[NV][V];
  float dot = 0.f, psum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * MS_THREADS + threadIdx.x) * V;
    if (c < cols) {
      const Vec16<T> a = ld16(p + c), b = ld16(g + c);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        pv[i][k] = to_f(a.v[k]);
        gv[i][k] = to_f(b.v[k]);
        dot = fmaf(pv[i][k], gv[i][k], dot);
        psum += pv[i][k];
      }
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) { pv[i][k] = 0.f; gv[i][k] = 0.f; }
    }
  }
  dot = block_reduce(dot, false, scratch);
  if (dsink_rows != nullptr) {  // the sink's probability is what the keys leave: d sink = -(1 - Σ P) · Σ P dP
    psum = block_reduce(psum, false, scratch);
    if (threadIdx.x == 0) dsink_rows[row] = -(1.f - psum) * dot;
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * MS_THREADS + threadIdx.x) * V;
    if (c < cols) {
      Vec16<T> o;
#pragma unroll
      for (int k = 0; k < V; ++k) o.v[k] = from_f<T>(scale * pv[i][k] * (gv[i][k] - dot));
      st16(d + c, o);
    }
  }
}

// Rows wider than the register budget: two passes over global memory (online maximum / sum, then the write).
template <typename T>
__global__ void __launch_bounds__(MS_THREADS) masked_softmax_fwd_stream_kernel(const T* __restrict__ S,
                                                                               const unsigned char* __restrict__ allowed,
                                                                               T* __restrict__ P, int cols,
                                                                               int mask_rows, float scale,
                                                                               const float* __restrict__ sink) {
  constexpr int V = Vec16<T>::N;
  __shared__ float scratch[MS_THREADS / 32];
  const long long row = blockIdx.x;
  const T* s = S + row * cols;
  T* p = P + row * cols;
  const unsigned char* a = allowed + (row % mask_rows) * (long long)cols;
  const float sk = sink != nullptr ? sink[row / mask_rows] : -INFINITY;
  float m = -INFINITY, l = 0.f;
  for (int c = threadIdx.x * V; c < cols; c += MS_THREADS * V) {
    const Vec16<T> v = ld16(s + c);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      if (a[c + k]) {
        const float x = to_f(v.v[k]) * scale;
        if (x > m) { l *= __expf(m - x); m = x; }
        l += __expf(x - m);
      }
    }
  }
  const float mb = fmaxf(block_reduce(m, true, scratch), sk);
  const bool empty = mb == -INFINITY;
  l = (m == -INFINITY) ? 0.f : l * __expf(m - mb);
  const float lb = block_reduce(l, false, scratch) + (empty ? 0.f : __expf(sk - mb));
  const float inv = empty ? 0.f : 1.f / lb;
  for (int c = threadIdx.x * V; c < cols; c += MS_THREADS * V) {
    const Vec16<T> v = ld16(s + c);
    Vec16<T> o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.v[k] = from_f<T>(a[c + k] ? __expf(to_f(v.v[k]) * scale - mb) * inv : 0.f);
    st16(p + c, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(MS_THREADS) masked_softmax_bwd_stream_kernel(const T* __restrict__ P,
                                                                               const T* __restrict__ dP,
                                                                               T* __restrict__ dS, int cols,
                                                                               float scale,
                                                                               float* __restrict__ dsink_rows) {
  constexpr int V = Vec16<T>::N;
  __shared__ float scratch[MS_THREADS / 32];
  const long long row = blockIdx.x;
  const T* p = P + row * cols;
  const T* g = dP + row * cols;
  T* d = dS + row * cols;
  float dot = 0.f, psum = 0.f;
  for (int c = threadIdx.x * V; c < cols; c += MS_THREADS * V) {
    const Vec16<T> a = ld16(p + c), b = ld16(g + c);
#pragma unroll
    for (int k = 0; k < V; ++k) { dot = fmaf(to_f(a.v[k]), to_f(b.v[k]), dot); psum += to_f(a.v[k]); }
  }
  dot = block_reduce(dot, false, scratch);
  if (dsink_rows != nullptr) {
    psum = block_reduce(psum, false, scratch);
    if (threadIdx.x == 0) dsink_rows[row] = -(1.f - psum) * dot;
  }
  for (int c = threadIdx.x * V; c < cols; c += MS_THREADS * V) {
    const Vec16<T> a = ld16(p + c), b = ld16(g + c);
    Vec16<T> o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.v[k] = from_f<T>(scale * to_f(a.v[k]) * (to_f(b.v[k]) - dot));
    st16(d + c, o);
  }
}

template <typename T>
void launch_fwd(const void* S, const void* allowed, void* P, long long rows, int cols, int mask_rows, float scale,
                const float* sink, cudaStream_t st) {
  // the row lives in registers: as few vectors per thread as the width needs (fewer registers, more rows in flight)
  const int per = MS_THREADS * Vec16<T>::N;
#define TB_MS_FWD(NV)                                                                                              \
  masked_softmax_fwd_kernel<T, NV><<<(unsigned)rows, MS_THREADS, 0, st>>>((const T*)S, (const unsigned char*)allowed, \
                                                                          (T*)P, cols, mask_rows, scale, sink)
  if (cols <= per) TB_MS_FWD(1);
  else if (cols <= 2 * per) TB_MS_FWD(2);
  else if (cols <= 4 * per) TB_MS_FWD(4);
  else if (cols <= MS_MAX_VECS * per) TB_MS_FWD(8);
  else
    masked_softmax_fwd_stream_kernel<T><<<(unsigned)rows, MS_THREADS, 0, st>>>(
        (const T*)S, (const unsigned char*)allowed, (T*)P, cols, mask_rows, scale, sink);
#undef TB_MS_FWD
}

template <typename T>
void launch_bwd(const void* P, const void* dP, void* dS, long long rows, int cols, float scale, float* dsink_rows,
                cudaStream_t st) {
  const int per = MS_THREADS * Vec16<T>::N;
#define TB_MS_BWD(NV)                                                                                            \
  masked_softmax_bwd_kernel<T, NV><<<(unsigned)rows, MS_THREADS, 0, st>>>((const T*)P, (const T*)dP, (T*)dS, cols, \
                                                                          scale, dsink_rows)
  if (cols <= per) TB_MS_BWD(1);
  else if (cols <= 2 * per) TB_MS_BWD(2);
  else if (cols <= 4 * per) TB_MS_BWD(4);
  else if (cols <= MS_MAX_VECS * per) TB_MS_BWD(8);
  else
    masked_softmax_bwd_stream_kernel<T><<<(unsigned)rows, MS_THREADS, 0, st>>>((const T*)P, (const T*)dP, (T*)dS, cols,
                                                                               scale, dsink_rows);
#undef TB_MS_BWD
}

}  // namespace

// S, P: [rows, cols] (dtype 0 fp32 / 1 bf16 / 2 fp16), allowed: [mask_rows, cols] bytes (0 = masked).
// cols a multiple of the 16-byte vector (8 for 16-bit types, 4 for fp32); rows of up to 256 * 8 vectors are held in
// registers, wider ones take two passes over global memory.
// sink: optional [rows / mask_rows] fp32, one logit per head that joins the denominator only (attention sink).
TB_API int tb_masked_softmax_fwd(const void* S, const void* allowed, void* P, long long rows, int cols, int mask_rows,
                                 float scale, const float* sink, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (cols <= 0 || mask_rows <= 0 || rows > 0x7fffffffLL) return TB_ERR_ARG;
  if (cols % (dtype == 0 ? 4 : 8)) return TB_ERR_ARG;
  if (dtype == 0) launch_fwd<float>(S, allowed, P, rows, cols, mask_rows, scale, sink, st);
  else if (dtype == 1) launch_fwd<__nv_bfloat16>(S, allowed, P, rows, cols, mask_rows, scale, sink, st);
  else if (dtype == 2) launch_fwd<__half>(S, allowed, P, rows, cols, mask_rows, scale, sink, st);
  else return TB_ERR_ARG;
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

// dsink_rows: optional [rows] fp32, the sink logit's gradient contribution of every row (the caller sums per head).
TB_API int tb_masked_softmax_bwd(const void* P, const void* dP, void* dS, long long rows, int cols, float scale,
                                 float* dsink_rows, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (cols <= 0 || rows > 0x7fffffffLL) return TB_ERR_ARG;
  if (cols % (dtype == 0 ? 4 : 8)) return TB_ERR_ARG;
  if (dtype == 0) launch_bwd<float>(P, dP, dS, rows, cols, scale, dsink_rows, st);
  else if (dtype == 1) launch_bwd<__nv_bfloat16>(P, dP, dS, rows, cols, scale, dsink_rows, st);
  else if (dtype == 2) launch_bwd<__half>(P, dP, dS, rows, cols, scale, dsink_rows, st);
  else return TB_ERR_ARG;
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
