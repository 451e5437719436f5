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

__device__ __forceinline__ float sigmoidf_(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                                                         T* __restrict__ out, const float* __restrict__ score,
                                                         long long rows, int H, long long in_pitch,
                                                         long long out_pitch, float limit) {
  constexpr int V = Vec16<T>::N;
  // a block walks whole rows (no index division); two vectors per thread are in flight per iteration
  auto act = [&](const Vec16<T>& gv, const Vec16<T>& uv, float sc) {
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
    return o;
  };
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* gp = gate + r * in_pitch;
    const T* upp = up + r * in_pitch;
    T* op = out + r * out_pitch;
    const float sc = score != nullptr ? score[r] : 1.f;
    int c = threadIdx.x * V;
    for (; c + (int)blockDim.x * V < H; c += 2 * blockDim.x * V) {
      const int c2 = c + blockDim.x * V;
      const Vec16<T> g1 = ld16(gp + c), u1 = ld16(upp + c), g2 = ld16(gp + c2), u2 = ld16(upp + c2);
      st16(op + c, act(g1, u1, sc));
      st16(op + c2, act(g2, u2, sc));
    }
    if (c < H) st16(op + c, act(ld16(gp + c), ld16(upp + c), sc));
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
    // a block per row (grid-stride): as many threads as half the row's vectors, between one warp and 256
    int block = ((H / V + 1) / 2 + 31) / 32 * 32;
    block = block < 32 ? 32 : (block > 256 ? 256 : block);
    const long long cap = 148LL * 16 * (256 / block);
    const int grid = (int)(rows < cap ? rows : cap);
    swiglu_fwd_kernel<T><<<grid, block, 0, st>>>((const T*)gate, (const T*)up, (T*)out, score, rows, H, in_pitch,
                                                 out_pitch, limit);
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
