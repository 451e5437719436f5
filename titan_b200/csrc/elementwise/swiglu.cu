// SwiGLU activation (+ optional clamp and per-row score) for sm_100a, forward and backward.
//
//   gate' = min(gate, L), up' = clamp(up, -L, L)   (L <= 0 disables clamping)
//   out   = silu(gate') * up' * score[row]          (score == nullptr → 1)
//
// Inputs are two row-major matrices with independent row pitches, so the same kernel serves
// separate w1/w3 outputs (pitch = H) and a fused [rows, 2H] buffer (gate = buf, up = buf + H,
// pitch = 2H).  Backward writes dgate/dup with the same pitches and, when scores are used,
// dscore[row] = sum_cols g * silu(gate') * up' (one warp per row, fixed order).
//
// Semantics follow the reference's expert activation (converters/kernels/gmm.py:87-104;
// models/deepseek_v4/moe.py:216-220: clamp gate from above, up on both sides, multiply by the
// routed score before the second grouped GEMM).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                                                         T* __restrict__ out, const float* __restrict__ score,
                                                         long long rows, int H, long long in_pitch,
                                                         long long out_pitch, float limit) {
  constexpr int V = Vec16<T>::N;
  const int vec_per_row = H / V;
  const long long total = rows * vec_per_row;
  for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < total;
       it += (long long)gridDim.x * blockDim.x) {
    const long long r = it / vec_per_row;
    const int c = (int)(it % vec_per_row) * V;
    Vec16<T> gv = ld16(gate + r * in_pitch + c), uv = ld16(up + r * in_pitch + c);
    const float sc = score != nullptr ? score[r] : 1.f;
    Vec16<T> o;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float g = to_f(gv.v[i]), u = to_f(uv.v[i]);
      if (limit > 0.f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
      }
      o.v[i] = from_f<T>(g * sigmoidf_(g) * u * sc);
    }
    st16(out + r * out_pitch + c, o);
  }
}

// one warp per row so dscore needs no atomics
template <typename T>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const T* __restrict__ gout, const T* __restrict__ gate,
                                                         const T* __restrict__ up, T* __restrict__ dgate,
                                                         T* __restrict__ dup, const float* __restrict__ score,
                                                         float* __restrict__ dscore, long long rows, int H,
                                                         long long in_pitch, long long out_pitch, float limit) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp0; r < rows; r += nwarps) {
    const float sc = score != nullptr ? score[r] : 1.f;
    float ds = 0.f;
    for (int c = lane * V; c < H; c += 32 * V) {
      Vec16<T> gv = ld16(gate + r * in_pitch + c), uv = ld16(up + r * in_pitch + c);
      Vec16<T> dv = ld16(gout + r * out_pitch + c);
      Vec16<T> og, ou;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float g = to_f(gv.v[i]), u = to_f(uv.v[i]);
        const float d = to_f(dv.v[i]);
        bool g_pass = true, u_pass = true;
        if (limit > 0.f) {
          g_pass = g <= limit;
          u_pass = (u >= -limit) && (u <= limit);
          g = fminf(g, limit);
          u = fminf(fmaxf(u, -limit), limit);
        }
        const float sg = sigmoidf_(g);
        const float act = g * sg;
        ds += d * act * u;
        const float dsilu = sg * (1.f + g * (1.f - sg));
        og.v[i] = from_f<T>(g_pass ? d * sc * u * dsilu : 0.f);
        ou.v[i] = from_f<T>(u_pass ? d * sc * act : 0.f);
      }
      st16(dgate + r * in_pitch + c, og);
      st16(dup + r * in_pitch + c, ou);
    }
    if (dscore != nullptr) {
      ds = warp_sum(ds);
      if (lane == 0) dscore[r] = ds;
    }
  }
}

int grid_for(long long work_items, int per_block) {
  long long g = (work_items + per_block - 1) / per_block;
  if (g > 148LL * 16) g = 148LL * 16;
  return g < 1 ? 1 : (int)g;
}
}  // namespace

#define TB_DISPATCH_DTYPE(dtype, ...)                    \
  switch (dtype) {                                       \
    case 0: { using T = float; __VA_ARGS__; break; }     \
    case 1: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case 2: { using T = __half; __VA_ARGS__; break; }    \
    default: return TB_ERR_ARG;                          \
  }

TB_API int tb_swiglu_fwd(const void* gate, const void* up, void* out, const float* score, long long rows, int H,
                         long long in_pitch, long long out_pitch, float limit, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  TB_DISPATCH_DTYPE(dtype, {
    constexpr int V = Vec16<T>::N;
    if (H % V != 0 || in_pitch % V != 0 || out_pitch % V != 0) return TB_ERR_ARG;
    swiglu_fwd_kernel<T><<<grid_for(rows * (H / V), 256), 256, 0, st>>>((const T*)gate, (const T*)up, (T*)out, score,
                                                                       rows, H, in_pitch, out_pitch, limit);
  });
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

TB_API int tb_swiglu_bwd(const void* gout, const void* gate, const void* up, void* dgate, void* dup,
                         const float* score, float* dscore, long long rows, int H, long long in_pitch,
                         long long out_pitch, float limit, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  TB_DISPATCH_DTYPE(dtype, {
    constexpr int V = Vec16<T>::N;
    if (H % V != 0 || in_pitch % V != 0 || out_pitch % V != 0) return TB_ERR_ARG;
    swiglu_bwd_kernel<T><<<grid_for(rows, 8), 256, 0, st>>>((const T*)gout, (const T*)gate, (const T*)up, (T*)dgate,
                                                           (T*)dup, score, dscore, rows, H, in_pitch, out_pitch,
                                                           limit);
  });
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
