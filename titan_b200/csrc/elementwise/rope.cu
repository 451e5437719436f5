// Rotary position embedding for sm_100a (memory-bound, 16-byte accesses, fp32 math).
//
// x: [B, S, H, D] contiguous.  Two layouts:
//   interleaved : pairs (x[2i], x[2i+1]) rotated by angle i; cache = [S_max, D/2, 2] fp32 (cos, sin)
//                 (this is `view_as_real` of the complex cache)
//   half        : pairs (x[i], x[i + D/2]); cache = [S_max, 2*D] fp32 = cos(D) | sin(D)
// `positions` (int64, [S] when pos_batch_stride == 0, else [B, S]) selects the cache row per token;
// nullptr means row = s.  `inverse` rotates by the negative angle, which is also the backward pass
// of the forward rotation (the transform is orthogonal), so one kernel serves fwd and bwd.
//
// Semantics follow the reference's RoPE op wrapper (converters/kernels/rope.py:68-201:
// interleave / half modes, inverse via negated sin, batch-shared positions).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

template <typename T, bool INTERLEAVED>
__global__ void __launch_bounds__(256) rope_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                   const float* __restrict__ cache,
                                                   const long long* __restrict__ positions, long long pos_bstride,
                                                   int B, int S, int H, int D, int cache_rows, float sin_sign,
                                                   int* __restrict__ status) {
  constexpr int V = Vec16<T>::N;
  // one work item = V consecutive elements (interleaved) or V elements of the low half + their partners (half)
  const int items_per_head = INTERLEAVED ? D / V : (D / 2) / V;
  const long long total = (long long)B * S * H * items_per_head;
  for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < total;
       it += (long long)gridDim.x * blockDim.x) {
    const int w = (int)(it % items_per_head);
    const long long tokh = it / items_per_head;
    const long long tok = tokh / H;  // b * S + s
    const int s = (int)(tok % S);
    const int b = (int)(tok / S);
    long long prow = s;
    if (positions != nullptr) prow = positions[(long long)b * pos_bstride + s];
    if (prow < 0 || prow >= cache_rows) {
      if (status != nullptr) atomicExch(status, TB_ERR_BOUNDS);
      continue;
    }
    const T* xp = x + tokh * D;
    T* yp = y + tokh * D;
    if constexpr (INTERLEAVED) {
      const int e0 = w * V;  // element offset in the head; pair index = e0/2 ...
      Vec16<T> xv = ld16(xp + e0);
      const float* c = cache + prow * D + e0;  // (cos, sin) per pair = D floats per row
      Vec16<T> o;
#pragma unroll
      for (int i = 0; i < V; i += 2) {
        const float cs = c[i], sn = c[i + 1] * sin_sign;
        const float a = to_f(xv.v[i]), bb = to_f(xv.v[i + 1]);
        o.v[i] = from_f<T>(a * cs - bb * sn);
        o.v[i + 1] = from_f<T>(a * sn + bb * cs);
      }
      st16(yp + e0, o);
    } else {
      const int e0 = w * V, half = D / 2;
      Vec16<T> lo = ld16(xp + e0), hi = ld16(xp + e0 + half);
      const float* cosr = cache + prow * 2 * D;
      const float* sinr = cosr + D;
      Vec16<T> olo, ohi;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float a = to_f(lo.v[i]), bb = to_f(hi.v[i]);
        // y_lo = a cos_lo - b sin_lo ; y_hi = b cos_hi + a sin_hi   (cos/sin duplicated over halves)
        olo.v[i] = from_f<T>(a * cosr[e0 + i] - bb * sinr[e0 + i] * sin_sign);
        ohi.v[i] = from_f<T>(bb * cosr[e0 + half + i] + a * sinr[e0 + half + i] * sin_sign);
      }
      st16(yp + e0, olo);
      st16(yp + e0 + half, ohi);
    }
  }
}

template <typename T>
int launch(const void* x, void* y, const float* cache, const long long* pos, long long pos_bstride, int B, int S,
           int H, int D, int cache_rows, int interleaved, int inverse, int* status, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  if (interleaved ? (D % V != 0) : ((D / 2) % V != 0 || D % 2 != 0)) return TB_ERR_ARG;
  const long long items = (long long)B * S * H * (interleaved ? D / V : D / 2 / V);
  if (items == 0) return 0;
  long long grid = (items + 255) / 256;
  if (grid > 148LL * 16) grid = 148LL * 16;
  const float sign = inverse ? -1.f : 1.f;
  if (interleaved)
    rope_kernel<T, true><<<(int)grid, 256, 0, st>>>((const T*)x, (T*)y, cache, pos, pos_bstride, B, S, H, D,
                                                    cache_rows, sign, status);
  else
    rope_kernel<T, false><<<(int)grid, 256, 0, st>>>((const T*)x, (T*)y, cache, pos, pos_bstride, B, S, H, D,
                                                     cache_rows, sign, status);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
}  // namespace

// dtype: 0 = fp32, 1 = bf16, 2 = fp16.  x and y may alias (in-place).
TB_API int tb_rope(const void* x, void* y, const float* cache, const long long* positions, long long pos_bstride,
                   int B, int S, int H, int D, int cache_rows, int interleaved, int inverse, int dtype, int* status,
                   cudaStream_t st) {
  switch (dtype) {
    case 0: return launch<float>(x, y, cache, positions, pos_bstride, B, S, H, D, cache_rows, interleaved, inverse, status, st);
    case 1: return launch<__nv_bfloat16>(x, y, cache, positions, pos_bstride, B, S, H, D, cache_rows, interleaved, inverse, status, st);
    case 2: return launch<__half>(x, y, cache, positions, pos_bstride, B, S, H, D, cache_rows, interleaved, inverse, status, st);
  }
  return TB_ERR_ARG;
}
