// Gated softmax pooling of the DeepSeek-V4 KV compressor (memory-bound, fp32).
//
//   out[b, c, j] = Σ_slot softmax_slot(score + ape) · kv      over the `ratio` tokens of block c
//
// With overlap (ratio 4) the projections are 2·d wide and a block pools 2·ratio candidates: the FIRST-half columns of
// the previous block's tokens (slots 0..r-1) and the SECOND-half columns of its own tokens (slots r..2r-1); block 0
// has no previous block.  Every input element therefore feeds exactly one output element, which makes the backward
// a pure elementwise pass once the forward has kept the log-sum-exp of each output:
//
//   p = exp(score + ape - lse[b,c,j]);  dkv = p · g;  dscore = p · (kv - out[b,c,j]) · g
//
// (first-half columns of the last block feed nothing: their gradients are zero).  The gradient of `ape` is the sum
// of dscore over batch and blocks, left to the caller as one reduction over the dscore tensor.
//
// Reference semantics: Compressor._forward_bsnd / _tnd of the reference's DeepSeek-V4 model (the eager pooling that
// its `compressor` kernel slot K23 replaces).
#include "../common/tb_common.cuh"

using namespace tb;

namespace {

// one thread per 4 consecutive output columns; candidates are read as float4 (coalesced along the columns)
__global__ void __launch_bounds__(256) pool_fwd_kernel(const float* __restrict__ kv, const float* __restrict__ score,
                                                       const float* __restrict__ ape, float* __restrict__ out,
                                                       float* __restrict__ lse, int B, int S, int r, int d,
                                                       int overlap) {
  const int C = S / r, d4 = d >> 2;
  const int width = overlap ? 2 * d : d;
  const long long total = (long long)B * C * d4;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(idx % d4) * 4;
    const int c = (int)((idx / d4) % C);
    const int b = (int)(idx / ((long long)d4 * C));
    float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    float l[4] = {0.f, 0.f, 0.f, 0.f}, acc[4] = {0.f, 0.f, 0.f, 0.f};
    const int halves = overlap ? 2 : 1;
    for (int h = 0; h < halves; ++h) {
      // overlap: h = 0 → previous block, first-half columns; h = 1 → this block, second-half columns
      const int blk = overlap ? (h == 0 ? c - 1 : c) : c;
      if (blk < 0) continue;
      const int col = overlap && h == 1 ? d + j : j;
      const float* kvp = kv + ((long long)b * S + (long long)blk * r) * width + col;
      const float* scp = score + ((long long)b * S + (long long)blk * r) * width + col;
      for (int i = 0; i < r; ++i) {
        const float4 s4 = *reinterpret_cast<const float4*>(scp + (long long)i * width);
        const float4 a4 = *reinterpret_cast<const float4*>(ape + (long long)i * width + col);
        const float4 k4 = *reinterpret_cast<const float4*>(kvp + (long long)i * width);
        const float s[4] = {s4.x + a4.x, s4.y + a4.y, s4.z + a4.z, s4.w + a4.w};
        const float k[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (s[u] > m[u]) {  // rescale the running sums (first candidate: exp(-inf) = 0)
            const float f = __expf(m[u] - s[u]);
            l[u] *= f; acc[u] *= f; m[u] = s[u];
          }
          const float p = __expf(s[u] - m[u]);
          l[u] += p; acc[u] = fmaf(p, k[u], acc[u]);
        }
      }
    }
    float4 o, ls;
    o.x = acc[0] / l[0]; o.y = acc[1] / l[1]; o.z = acc[2] / l[2]; o.w = acc[3] / l[3];
    ls.x = m[0] + __logf(l[0]); ls.y = m[1] + __logf(l[1]); ls.z = m[2] + __logf(l[2]); ls.w = m[3] + __logf(l[3]);
    const long long off = ((long long)b * C + c) * d + j;
    *reinterpret_cast<float4*>(out + off) = o;
    *reinterpret_cast<float4*>(lse + off) = ls;
  }
}

// one thread per 4 consecutive input columns of one token
__global__ void __launch_bounds__(256) pool_bwd_kernel(const float* __restrict__ kv, const float* __restrict__ score,
                                                       const float* __restrict__ ape, const float* __restrict__ out,
                                                       const float* __restrict__ lse, const float* __restrict__ gout,
                                                       float* __restrict__ dkv, float* __restrict__ dscore, int B,
                                                       int S, int r, int d, int overlap) {
  const int C = S / r;
  const int width = overlap ? 2 * d : d;
  const int w4 = width >> 2;
  const long long total = (long long)B * S * w4;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int col = (int)(idx % w4) * 4;
    const int t = (int)((idx / w4) % S);
    const int b = (int)(idx / ((long long)w4 * S));
    const int blk = t / r, i = t - blk * r;
    int c = blk, j = col;
    if (overlap) {
      if (col < d) c = blk + 1;  // first half feeds the NEXT block
      else j = col - d;
    }
    const long long in_off = ((long long)b * S + t) * width + col;
    float4 gk = make_float4(0.f, 0.f, 0.f, 0.f), gs = gk;
    if (c < C) {
      const long long o_off = ((long long)b * C + c) * d + j;
      const float4 s4 = *reinterpret_cast<const float4*>(score + in_off);
      const float4 a4 = *reinterpret_cast<const float4*>(ape + (long long)i * width + col);
      const float4 k4 = *reinterpret_cast<const float4*>(kv + in_off);
      const float4 o4 = *reinterpret_cast<const float4*>(out + o_off);
      const float4 l4 = *reinterpret_cast<const float4*>(lse + o_off);
      const float4 g4 = *reinterpret_cast<const float4*>(gout + o_off);
      const float p0 = __expf(s4.x + a4.x - l4.x), p1 = __expf(s4.y + a4.y - l4.y);
      const float p2 = __expf(s4.z + a4.z - l4.z), p3 = __expf(s4.w + a4.w - l4.w);
      gk = make_float4(p0 * g4.x, p1 * g4.y, p2 * g4.z, p3 * g4.w);
      gs = make_float4(gk.x * (k4.x - o4.x), gk.y * (k4.y - o4.y), gk.z * (k4.z - o4.z), gk.w * (k4.w - o4.w));
    }
    *reinterpret_cast<float4*>(dkv + in_off) = gk;
    *reinterpret_cast<float4*>(dscore + in_off) = gs;
  }
}

int grid_for(long long total) {
  long long g = (total + 255) / 256;
  if (g > 148LL * 16) g = 148LL * 16;
  return g < 1 ? 1 : (int)g;
}

}  // namespace

// kv, score [B, S, width] fp32 (width = d, or 2·d with overlap); ape [ratio, width]; out, lse [B, S / ratio, d].
TB_API int tb_compressor_pool_fwd(const float* kv, const float* score, const float* ape, float* out, float* lse, int B,
                                  int S, int ratio, int d, int overlap, cudaStream_t st) {
  if (B <= 0 || S <= 0 || ratio <= 0 || S % ratio || d <= 0 || d % 4) return TB_ERR_ARG;
  const long long total = (long long)B * (S / ratio) * (d / 4);
  pool_fwd_kernel<<<grid_for(total), 256, 0, st>>>(kv, score, ape, out, lse, B, S, ratio, d, overlap);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

// gout [B, S / ratio, d]; dkv, dscore [B, S, width] (every element is written)
TB_API int tb_compressor_pool_bwd(const float* kv, const float* score, const float* ape, const float* out,
                                  const float* lse, const float* gout, float* dkv, float* dscore, int B, int S,
                                  int ratio, int d, int overlap, cudaStream_t st) {
  if (B <= 0 || S <= 0 || ratio <= 0 || S % ratio || d <= 0 || d % 4) return TB_ERR_ARG;
  const long long total = (long long)B * S * ((overlap ? 2 * d : d) / 4);
  pool_bwd_kernel<<<grid_for(total), 256, 0, st>>>(kv, score, ape, out, lse, gout, dkv, dscore, B, S, ratio, d,
                                                   overlap);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
