// Hyper-connection (mHC) kernels for sm_100a: hc = 4 residual streams of width D per token, bf16 streams, fp32 math.
//
//   pre   : rstd = rsqrt(mean(x^2) + norm_eps) over the 4*D stream values;  mixes = raw * rstd  (raw = x_flat . fn^T is
//           a skinny GEMM and runs on the tensor cores before this kernel; it arrives as fp32 [T, ld] with a bf16
//           hi/lo split of fn: columns 0..23 hold x.fn_hi, columns 32..55 hold x.fn_lo)
//           pre[m]  = sigmoid(mixes[m]   * s0 + b[m])   + eps
//           post[m] = 2 * sigmoid(mixes[4+m] * s1 + b[4+m])
//           comb    = Sinkhorn(softmax_n(mixes[8+4m+n] * s2 + b[8+4m+n]) + eps):  one column pass, then iters-1
//                     (row, column) passes, every pass  c <- c / (sum + eps)
//           y[d]    = sum_m pre[m] * x[m, d]
//   post  : out[n, d] = post[n] * y[d] + sum_m comb[m, n] * res[m, d]
//
// One CTA per token keeps the token's 4*D values in registers: x is read once per kernel, the RMS statistic and
// the weighted stream sum need no second pass.  The 4x4 Sinkhorn runs on 16 lanes of warp 0 (lane = 4*m + n; row
// sums = xor-shuffles 1, 2; column sums = xor-shuffles 4, 8); the backward keeps every pass's output and inverse
// denominator in shared memory (40 x 16 x 2 floats) and walks the passes in reverse.
//
// Semantics: HcSplitSinkhorn / HcPre / HcPost of the reference (models/deepseek_v4/model.py:986-1075); the reference's
// fused ops are npu_mhc_pre / npu_mhc_post (converters/kernels/mhc_prepost.py).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int HC = 4;
constexpr int MIX = 24;
constexpr int NT = 256;
constexpr int NW = NT / 32;
constexpr int MAX_PASSES = 2 * 64;  // Sinkhorn passes kept for backward (iters <= 64)

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + __expf(-z)); }

// block-wide sums of N values per thread; result valid in every thread.  `red` holds N * NW floats.
template <int N>
__device__ __forceinline__ void block_sum(float (&v)[N], float* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < N; ++i) {
    v[i] = warp_sum(v[i]);
    if (lane == 0) red[i * NW + warp] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) s += red[i * NW + w];
    v[i] = s;
  }
  __syncthreads();  // `red` may be reused
}

__device__ __forceinline__ float row_sum16(float v) {  // over n (lane bits 0, 1)
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}
__device__ __forceinline__ float col_sum16(float v) {  // over m (lane bits 2, 3)
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  return v;
}

// Forward Sinkhorn on the 16 lanes of a warp (lanes 16..31 mirror 0..15).  `keep_y`, `keep_inv` (or nullptr):
// per-pass outputs and inverse denominators for the backward, indexed [pass][lane & 15]; returns the element.
__device__ __forceinline__ float sinkhorn_fwd(float z, int iters, float eps, float* keep_y, float* keep_inv,
                                              float* p_out) {
  const int l = threadIdx.x & 15;
  // softmax over n
  float mx = z;
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  const float e = __expf(z - mx);
  const float p = e / row_sum16(e);
  if (p_out) *p_out = p;
  float c = p + eps;
  int pass = 0;
  {  // first column pass
    const float inv = 1.f / (col_sum16(c) + eps);
    c *= inv;
    if (keep_y) { keep_y[pass * 16 + l] = c; keep_inv[pass * 16 + l] = inv; }
    ++pass;
  }
  for (int it = 1; it < iters; ++it) {
    float inv = 1.f / (row_sum16(c) + eps);
    c *= inv;
    if (keep_y) { keep_y[pass * 16 + l] = c; keep_inv[pass * 16 + l] = inv; }
    ++pass;
    inv = 1.f / (col_sum16(c) + eps);
    c *= inv;
    if (keep_y) { keep_y[pass * 16 + l] = c; keep_inv[pass * 16 + l] = inv; }
    ++pass;
  }
  return c;
}

// ---------------------------------------------------------------------------------------------------- pre forward
template <int CH>
__global__ void __launch_bounds__(NT) mhc_pre_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                         const float* __restrict__ raw, long long ld_raw,
                                                         const float* __restrict__ scale,
                                                         const float* __restrict__ base, int iters, float hc_eps,
                                                         float norm_eps, int D, __nv_bfloat16* __restrict__ y,
                                                         float* __restrict__ post_out, float* __restrict__ comb_out,
                                                         float* __restrict__ pre_out, float* __restrict__ rstd_out) {
  using V = Vec16<__nv_bfloat16>;
  __shared__ float red[NW];
  __shared__ float s_pre[HC];
  const long long t = blockIdx.x;
  const __nv_bfloat16* xt = x + t * HC * (long long)D;
  V xv[HC][CH];
  float ss = 0.f;
#pragma unroll
  for (int m = 0; m < HC; ++m)
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const int c = (j * NT + threadIdx.x) * 8;
      if (c < D) {
        xv[m][j] = ld16(xt + (long long)m * D + c);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float f = to_f(xv[m][j].v[i]);
          ss += f * f;
        }
      }
    }
  float sv[1] = {ss};
  block_sum<1>(sv, red);
  const float rstd = rsqrtf(sv[0] / (float)(HC * D) + norm_eps);
  if (threadIdx.x < 32) {
    const int l = threadIdx.x & 15;
    const float* r = raw + t * ld_raw;
    // pre / post on lanes 0..3 / 4..7 (computed by every lane for its index, written by the owners)
    const float mixv = (r[l < 8 ? l : 0] + r[32 + (l < 8 ? l : 0)]) * rstd;
    if (threadIdx.x < 4) {
      const float pre = sigmoidf_(mixv * scale[0] + base[l]) + hc_eps;
      s_pre[l] = pre;
      pre_out[t * HC + l] = pre;
    } else if (threadIdx.x < 8) {
      post_out[t * HC + (l - 4)] = 2.f * sigmoidf_(mixv * scale[1] + base[l]);
    }
    const float mc = (r[8 + l] + r[32 + 8 + l]) * rstd;
    const float c = sinkhorn_fwd(mc * scale[2] + base[8 + l], iters, hc_eps, nullptr, nullptr, nullptr);
    if (threadIdx.x < 16) comb_out[t * 16 + l] = c;
    if (threadIdx.x == 0) rstd_out[t] = rstd;
  }
  __syncthreads();
  const float p0 = s_pre[0], p1 = s_pre[1], p2 = s_pre[2], p3 = s_pre[3];
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = (j * NT + threadIdx.x) * 8;
    if (c < D) {
      V o;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        o.v[i] = from_f<__nv_bfloat16>(p0 * to_f(xv[0][j].v[i]) + p1 * to_f(xv[1][j].v[i]) +
                                       p2 * to_f(xv[2][j].v[i]) + p3 * to_f(xv[3][j].v[i]));
      st16(y + t * D + c, o);
    }
  }
}

// ---------------------------------------------------------------------------------------------------- pre backward
// Stage 1 (per token): dpre[m] = gy . x[m]; back through sigmoid / Sinkhorn / softmax to dz[24] (gradient with
// respect to mixes*scale + base); G = dz * scale_k * rstd (bf16, row of the dx / dfn GEMM operands, padded to 64);
// coef = -(sum_j dz_j * scale_k * raw_j) * rstd^3 / (4 D)   (the RMS statistic's share of dx).
template <int CH>
__global__ void __launch_bounds__(NT) mhc_pre_bwd_small_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gy, const float* __restrict__ raw,
    long long ld_raw, const float* __restrict__ scale, const float* __restrict__ base, const float* __restrict__ rstd_in,
    const float* __restrict__ pre_in, const float* __restrict__ gpost, const float* __restrict__ gcomb, int iters,
    float hc_eps, int D, float* __restrict__ dz_out, float* __restrict__ mixes_out, __nv_bfloat16* __restrict__ G,
    float* __restrict__ coef_out) {
  using V = Vec16<__nv_bfloat16>;
  __shared__ float red[HC * NW];
  __shared__ float keep_y[MAX_PASSES * 16];
  __shared__ float keep_inv[MAX_PASSES * 16];
  __shared__ float s_c[MIX];
  const long long t = blockIdx.x;
  const __nv_bfloat16* xt = x + t * HC * (long long)D;
  float dots[HC] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = (j * NT + threadIdx.x) * 8;
    if (c < D) {
      const V g = ld16(gy + t * D + c);
#pragma unroll
      for (int m = 0; m < HC; ++m) {
        const V xv = ld16(xt + (long long)m * D + c);
#pragma unroll
        for (int i = 0; i < 8; ++i) dots[m] += to_f(g.v[i]) * to_f(xv.v[i]);
      }
    }
  }
  block_sum<HC>(dots, red);
  if (threadIdx.x < 32) {
    const int l = threadIdx.x & 15;
    const float rstd = rstd_in[t];
    const float* r = raw + t * ld_raw;
    float dz_small = 0.f, mix_small = 0.f;
    if (l < 8) {
      mix_small = (r[l] + r[32 + l]) * rstd;
      if (l < 4) {
        const float sg = pre_in[t * HC + l] - hc_eps;  // sigmoid value
        dz_small = dots[l] * sg * (1.f - sg);
      } else {
        const float sg = sigmoidf_(mix_small * scale[1] + base[l]);
        dz_small = gpost[t * HC + (l - 4)] * 2.f * sg * (1.f - sg);
      }
    }
    // Sinkhorn: forward with kept passes, then the passes in reverse
    const float mc = (r[8 + l] + r[32 + 8 + l]) * rstd;
    float p;
    sinkhorn_fwd(mc * scale[2] + base[8 + l], iters, hc_eps, keep_y, keep_inv, &p);
    __syncwarp();
    float g = gcomb[t * 16 + l];
    int pass = 2 * iters - 2;  // index of the last pass (a column pass)
    for (; pass >= 0; --pass) {
      const float yv = keep_y[pass * 16 + l], inv = keep_inv[pass * 16 + l];
      const bool column = (pass & 1) == 0;  // pass 0 and every even pass normalise columns
      const float gy_sum = column ? col_sum16(g * yv) : row_sum16(g * yv);
      g = (g - gy_sum) * inv;
    }
    const float gp_sum = row_sum16(g * p);  // softmax over n; the +eps is a constant shift
    const float dz_c = p * (g - gp_sum);
    if (threadIdx.x < 16) {
      dz_out[t * MIX + 8 + l] = dz_c;
      mixes_out[t * MIX + 8 + l] = mc;
      s_c[8 + l] = dz_c * scale[2];
      if (l < 8) {
        dz_out[t * MIX + l] = dz_small;
        mixes_out[t * MIX + l] = mix_small;
        s_c[l] = dz_small * scale[l < 4 ? 0 : 1];
      }
    }
    __syncwarp();
    if (threadIdx.x < 32) {
      // G row (64 wide, zero padded) and the coefficient of x
      const float dm0 = threadIdx.x < MIX ? s_c[threadIdx.x] : 0.f;  // gradient with respect to mixes
      G[t * 64 + threadIdx.x] = from_f<__nv_bfloat16>(dm0 * rstd);
      G[t * 64 + 32 + threadIdx.x] = from_f<__nv_bfloat16>(0.f);
      float acc = threadIdx.x < MIX ? dm0 * (r[threadIdx.x] + r[32 + threadIdx.x]) : 0.f;
      acc = warp_sum(acc);
      if (threadIdx.x == 0) coef_out[t] = -acc * rstd * rstd * rstd / (float)(HC * D);
    }
  }
}

// Stage 2: dx[m, d] = pre[m] * gy[d] + coef * x[m, d] + dxf[m, d]   (dxf = G . fn, from the tensor cores)
template <int CH>
__global__ void __launch_bounds__(NT) mhc_pre_bwd_dx_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ gy,
                                                            const __nv_bfloat16* __restrict__ dxf,
                                                            const float* __restrict__ pre_in,
                                                            const float* __restrict__ coef_in, int D,
                                                            __nv_bfloat16* __restrict__ dx) {
  using V = Vec16<__nv_bfloat16>;
  const long long t = blockIdx.x;
  const float coef = coef_in[t];
  float pre[HC];
#pragma unroll
  for (int m = 0; m < HC; ++m) pre[m] = pre_in[t * HC + m];
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = (j * NT + threadIdx.x) * 8;
    if (c < D) {
      const V g = ld16(gy + t * D + c);
#pragma unroll
      for (int m = 0; m < HC; ++m) {
        const long long off = (t * HC + m) * (long long)D + c;
        const V xv = ld16(x + off), f = ld16(dxf + off);
        V o;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          o.v[i] = from_f<__nv_bfloat16>(pre[m] * to_f(g.v[i]) + coef * to_f(xv.v[i]) + to_f(f.v[i]));
        st16(dx + off, o);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------- post
template <int CH>
__global__ void __launch_bounds__(NT) mhc_post_fwd_kernel(const __nv_bfloat16* __restrict__ y,
                                                          const __nv_bfloat16* __restrict__ res,
                                                          const float* __restrict__ post,
                                                          const float* __restrict__ comb, int D,
                                                          __nv_bfloat16* __restrict__ out) {
  using V = Vec16<__nv_bfloat16>;
  const long long t = blockIdx.x;
  float po[HC], cb[HC][HC];
#pragma unroll
  for (int n = 0; n < HC; ++n) po[n] = post[t * HC + n];
#pragma unroll
  for (int m = 0; m < HC; ++m)
#pragma unroll
    for (int n = 0; n < HC; ++n) cb[m][n] = comb[t * 16 + m * HC + n];
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = (j * NT + threadIdx.x) * 8;
    if (c < D) {
      const V yv = ld16(y + t * D + c);
      V r[HC];
#pragma unroll
      for (int m = 0; m < HC; ++m) r[m] = ld16(res + (t * HC + m) * (long long)D + c);
#pragma unroll
      for (int n = 0; n < HC; ++n) {
        V o;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float a = po[n] * to_f(yv.v[i]);
#pragma unroll
          for (int m = 0; m < HC; ++m) a += cb[m][n] * to_f(r[m].v[i]);
          o.v[i] = from_f<__nv_bfloat16>(a);
        }
        st16(out + (t * HC + n) * (long long)D + c, o);
      }
    }
  }
}

// dy[d] = sum_n post[n] go[n,d];  dres[m,d] = sum_n comb[m,n] go[n,d];  dpost[n] = go[n].y;  dcomb[m,n] = res[m].go[n]
template <int CH>
__global__ void __launch_bounds__(NT) mhc_post_bwd_kernel(const __nv_bfloat16* __restrict__ go,
                                                          const __nv_bfloat16* __restrict__ y,
                                                          const __nv_bfloat16* __restrict__ res,
                                                          const float* __restrict__ post,
                                                          const float* __restrict__ comb, int D,
                                                          __nv_bfloat16* __restrict__ dy,
                                                          __nv_bfloat16* __restrict__ dres, float* __restrict__ dpost,
                                                          float* __restrict__ dcomb) {
  using V = Vec16<__nv_bfloat16>;
  __shared__ float red[20 * NW];
  const long long t = blockIdx.x;
  float po[HC], cb[HC][HC];
#pragma unroll
  for (int n = 0; n < HC; ++n) po[n] = post[t * HC + n];
#pragma unroll
  for (int m = 0; m < HC; ++m)
#pragma unroll
    for (int n = 0; n < HC; ++n) cb[m][n] = comb[t * 16 + m * HC + n];
  float acc[20];
#pragma unroll
  for (int i = 0; i < 20; ++i) acc[i] = 0.f;
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = (j * NT + threadIdx.x) * 8;
    if (c < D) {
      const V yv = ld16(y + t * D + c);
      V g[HC], r[HC];
#pragma unroll
      for (int n = 0; n < HC; ++n) {
        g[n] = ld16(go + (t * HC + n) * (long long)D + c);
        r[n] = ld16(res + (t * HC + n) * (long long)D + c);
      }
      V o;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float a = 0.f;
#pragma unroll
        for (int n = 0; n < HC; ++n) a += po[n] * to_f(g[n].v[i]);
        o.v[i] = from_f<__nv_bfloat16>(a);
      }
      st16(dy + t * D + c, o);
#pragma unroll
      for (int m = 0; m < HC; ++m) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float a = 0.f;
#pragma unroll
          for (int n = 0; n < HC; ++n) a += cb[m][n] * to_f(g[n].v[i]);
          o.v[i] = from_f<__nv_bfloat16>(a);
        }
        st16(dres + (t * HC + m) * (long long)D + c, o);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float yf = to_f(yv.v[i]);
#pragma unroll
        for (int n = 0; n < HC; ++n) {
          const float gf = to_f(g[n].v[i]);
          acc[n] += gf * yf;
#pragma unroll
          for (int m = 0; m < HC; ++m) acc[4 + m * HC + n] += to_f(r[m].v[i]) * gf;
        }
      }
    }
  }
  block_sum<20>(acc, red);
  if (threadIdx.x < 4) dpost[t * HC + threadIdx.x] = acc[threadIdx.x];
  else if (threadIdx.x < 20) dcomb[t * 16 + (threadIdx.x - 4)] = acc[threadIdx.x];
}

int ch_for(int D) {
  const int vecs = (D / 8 + NT - 1) / NT;
  return vecs <= 1 ? 1 : (vecs <= 2 ? 2 : (vecs <= 4 ? 4 : 0));
}

#define TB_MHC_DISPATCH(KERNEL, ...)                                            \
  do {                                                                          \
    switch (ch_for(D)) {                                                        \
      case 1: KERNEL<1><<<(unsigned)T, NT, 0, st>>>(__VA_ARGS__); break;        \
      case 2: KERNEL<2><<<(unsigned)T, NT, 0, st>>>(__VA_ARGS__); break;        \
      case 4: KERNEL<4><<<(unsigned)T, NT, 0, st>>>(__VA_ARGS__); break;        \
      default: return TB_ERR_ARG;                                               \
    }                                                                           \
    TB_CUDA_CHECK(cudaGetLastError());                                          \
    tb_note_launch(1);                                                          \
  } while (0)

bool bad(long long T, int D, int iters) { return T < 0 || D < 8 || D % 8 != 0 || D > 8192 || iters < 1 || iters > 64; }
}  // namespace

// x: [T, 4, D] bf16; raw: [T, ld_raw] fp32 (>= 56 columns, see header); scale [3], base [24] fp32.
TB_API int tb_mhc_pre_fwd(const void* x, const float* raw, long long ld_raw, const float* scale, const float* base,
                          int iters, float hc_eps, float norm_eps, long long T, int D, void* y, float* post,
                          float* comb, float* pre, float* rstd, cudaStream_t st) {
  if (T == 0) return 0;
  if (bad(T, D, iters) || ld_raw < 56) return TB_ERR_ARG;
  TB_MHC_DISPATCH(mhc_pre_fwd_kernel, (const __nv_bfloat16*)x, raw, ld_raw, scale, base, iters, hc_eps, norm_eps, D,
                  (__nv_bfloat16*)y, post, comb, pre, rstd);
  return 0;
}

// Outputs: dz, mixes [T, 24] fp32 (for the scale / base gradients), G [T, 64] bf16, coef [T] fp32.
TB_API int tb_mhc_pre_bwd_small(const void* x, const void* gy, const float* raw, long long ld_raw, const float* scale,
                                const float* base, const float* rstd, const float* pre, const float* gpost,
                                const float* gcomb, int iters, float hc_eps, long long T, int D, float* dz,
                                float* mixes, void* G, float* coef, cudaStream_t st) {
  if (T == 0) return 0;
  if (bad(T, D, iters) || ld_raw < 56) return TB_ERR_ARG;
  TB_MHC_DISPATCH(mhc_pre_bwd_small_kernel, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gy, raw, ld_raw, scale, base,
                  rstd, pre, gpost, gcomb, iters, hc_eps, D, dz, mixes, (__nv_bfloat16*)G, coef);
  return 0;
}

TB_API int tb_mhc_pre_bwd_dx(const void* x, const void* gy, const void* dxf, const float* pre, const float* coef,
                             long long T, int D, void* dx, cudaStream_t st) {
  if (T == 0) return 0;
  if (bad(T, D, 1)) return TB_ERR_ARG;
  TB_MHC_DISPATCH(mhc_pre_bwd_dx_kernel, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gy, (const __nv_bfloat16*)dxf,
                  pre, coef, D, (__nv_bfloat16*)dx);
  return 0;
}

TB_API int tb_mhc_post_fwd(const void* y, const void* res, const float* post, const float* comb, long long T, int D,
                           void* out, cudaStream_t st) {
  if (T == 0) return 0;
  if (bad(T, D, 1)) return TB_ERR_ARG;
  TB_MHC_DISPATCH(mhc_post_fwd_kernel, (const __nv_bfloat16*)y, (const __nv_bfloat16*)res, post, comb, D,
                  (__nv_bfloat16*)out);
  return 0;
}

TB_API int tb_mhc_post_bwd(const void* go, const void* y, const void* res, const float* post, const float* comb,
                           long long T, int D, void* dy, void* dres, float* dpost, float* dcomb, cudaStream_t st) {
  if (T == 0) return 0;
  if (bad(T, D, 1)) return TB_ERR_ARG;
  TB_MHC_DISPATCH(mhc_post_bwd_kernel, (const __nv_bfloat16*)go, (const __nv_bfloat16*)y, (const __nv_bfloat16*)res,
                  post, comb, D, (__nv_bfloat16*)dy, (__nv_bfloat16*)dres, dpost, dcomb);
  return 0;
}
