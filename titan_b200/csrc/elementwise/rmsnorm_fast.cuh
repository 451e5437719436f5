// Register-resident RMSNorm kernels: every element is read from memory exactly once.
//
//   forward   1, 2, 4 or 8 warps per row, the whole row lives in registers (at most 4-8 16-byte vectors per lane);
//             all loads of a row are issued back to back, statistics by warp shuffle (+ one barrier when warps
//             share a row), one store pass.
//   backward  (a) dim <= 512 elements of a 16-bit type: one warp per row, dw accumulators in registers
//                 (CH*V per lane), a cross-warp reduction through shared memory at the end of the CTA;
//             (b) larger rows: one CTA (NT threads) per group of R rows; thread t owns CH vectors of every row, so
//                 its dw accumulators (CH*V floats) stay in registers and its R rows of g and x are in flight
//                 together (R*CH = 2 keeps the kernel at 64 registers: two 512-thread CTAs per SM); the R row dot
//                 products are reduced with one __syncthreads per group.
//             Both write one fp32 partial row per CTA into dw_partial[grid, dim]; a second kernel reduces the
//             partial rows in a fixed order, so results are bitwise reproducible.
//
// Occupancy is the point of this layout: no dynamic shared memory (the previous design kept 16 KB of accumulators
// per warp and ran 8 warps per SM at 12 % active warps), 32+ warps per SM, 128+ KB of loads in flight per SM.
#pragma once
#include "../common/tb_common.cuh"

namespace tb_rms {
using namespace tb;

// WPR warps share a row (CH vectors per lane); a CTA of 8 warps covers 8 / WPR rows.
template <typename T, int CH, int WPR>
__global__ void __launch_bounds__(256) fwd_rowreg_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                         T* __restrict__ y, float* __restrict__ rstd_out, int rows,
                                                         int dim, float eps) {
  constexpr int V = Vec16<T>::N;
  constexpr int RPC = 8 / WPR;  // rows per CTA
  __shared__ float red[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = warp % WPR;  // which part of the row this warp holds
  const int row = blockIdx.x * RPC + warp / WPR;
  const bool live = row < rows;
  const T* xr = x + (size_t)(live ? row : 0) * dim;
  Vec16<T> xv[CH];
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = ((j * WPR + sub) * 32 + lane) * V;
    if (live && c < dim) {
      xv[j] = ld16(xr + c);
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) xv[j].v[i] = from_f<T>(0.f);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < CH; ++j)
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float f = to_f(xv[j].v[i]);
      ss += f * f;
    }
  ss = warp_sum(ss);
  if (WPR > 1) {
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int k = 0; k < WPR; ++k) ss += red[(warp / WPR) * WPR + k];
  }
  if (!live) return;
  const float rstd = rsqrtf(ss / (float)dim + eps);
  if (lane == 0 && sub == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
  T* yr = y + (size_t)row * dim;
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = ((j * WPR + sub) * 32 + lane) * V;
    if (c < dim) {
      const Vec16<T> wv = ld16(w + c);
      Vec16<T> o;
#pragma unroll
      for (int i = 0; i < V; ++i) o.v[i] = from_f<T>(to_f(xv[j].v[i]) * rstd * to_f(wv.v[i]));
      st16(yr + c, o);
    }
  }
}

// (a) warp per row, 8 warps per CTA
template <typename T, int CH>
__global__ void __launch_bounds__(256) bwd_warp_kernel(const T* __restrict__ g, const T* __restrict__ x,
                                                       const T* __restrict__ w, const float* __restrict__ rstd_in,
                                                       T* __restrict__ dx, float* __restrict__ dw_partial, int rows,
                                                       int dim) {
  constexpr int V = Vec16<T>::N;
  constexpr int WARPS = 8;
  __shared__ float red[WARPS][CH * 32 * V + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float acc[CH][V];
  float wf[CH][V];
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = (j * 32 + lane) * V;
    Vec16<T> wv;
    if (c < dim) wv = ld16(w + c);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      acc[j][i] = 0.f;
      wf[j][i] = c < dim ? to_f(wv.v[i]) : 0.f;
    }
  }
  for (int row = blockIdx.x * WARPS + warp; row < rows; row += gridDim.x * WARPS) {
    const T* gr = g + (size_t)row * dim;
    const T* xr = x + (size_t)row * dim;
    Vec16<T> gv[CH], xv[CH];
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const int c = (j * 32 + lane) * V;
      if (c < dim) {
        gv[j] = ld16(gr + c);
        xv[j] = ld16(xr + c);
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) gv[j].v[i] = xv[j].v[i] = from_f<T>(0.f);
      }
    }
    const float rstd = rstd_in[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < CH; ++j)
#pragma unroll
      for (int i = 0; i < V; ++i) dot += to_f(gv[j].v[i]) * wf[j][i] * to_f(xv[j].v[i]);
    dot = warp_sum(dot);
    const float k = dot * rstd * rstd / (float)dim;
    T* dr = dx + (size_t)row * dim;
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const int c = (j * 32 + lane) * V;
      Vec16<T> o;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float gf = to_f(gv[j].v[i]), xf = to_f(xv[j].v[i]);
        o.v[i] = from_f<T>(rstd * (gf * wf[j][i] - xf * k));
        acc[j][i] += gf * xf * rstd;
      }
      if (c < dim) st16(dr + c, o);
    }
  }
#pragma unroll
  for (int j = 0; j < CH; ++j)
#pragma unroll
    for (int i = 0; i < V; ++i) red[warp][(j * 32 + lane) * V + i] = acc[j][i];
  __syncthreads();
  float* out = dw_partial + (size_t)blockIdx.x * dim;
  for (int c = threadIdx.x; c < dim; c += WARPS * 32) {
    float s = 0.f;
#pragma unroll
    for (int wi = 0; wi < WARPS; ++wi) s += red[wi][c];
    out[c] = s;
  }
}

// (b) CTA of NT threads per group of R rows
template <typename T, int NT, int CH, int R>
__global__ void __launch_bounds__(NT, (CH * R <= 2) ? 1024 / NT : 1) bwd_cta_kernel(const T* __restrict__ g, const T* __restrict__ x,
                                                     const T* __restrict__ w, const float* __restrict__ rstd_in,
                                                     T* __restrict__ dx, float* __restrict__ dw_partial, int rows,
                                                     int dim) {
  constexpr int V = Vec16<T>::N;
  constexpr int NW = NT / 32;
  __shared__ float red[2][R][NW];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float acc[CH][V];
  float wf[CH][V];
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = (j * NT + threadIdx.x) * V;
    Vec16<T> wv;
    if (c < dim) wv = ld16(w + c);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      acc[j][i] = 0.f;
      wf[j][i] = c < dim ? to_f(wv.v[i]) : 0.f;
    }
  }
  int it = 0;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R, ++it) {
    Vec16<T> gv[R][CH], xv[R][CH];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int c = (j * NT + threadIdx.x) * V;
        if (row < rows && c < dim) {
          gv[r][j] = ld16(g + (size_t)row * dim + c);
          xv[r][j] = ld16(x + (size_t)row * dim + c);
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) gv[r][j].v[i] = xv[r][j].v[i] = from_f<T>(0.f);
        }
      }
    }
    float dot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < CH; ++j)
#pragma unroll
        for (int i = 0; i < V; ++i) d += to_f(gv[r][j].v[i]) * wf[j][i] * to_f(xv[r][j].v[i]);
      d = warp_sum(d);
      if (lane == 0) red[it & 1][r][warp] = d;
    }
    __syncthreads();  // the other buffer is free again: its readers passed the barrier of the previous group
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float d = 0.f;
#pragma unroll
      for (int wi = 0; wi < NW; ++wi) d += red[it & 1][r][wi];
      dot[r] = d;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
      if (row >= rows) continue;
      const float rstd = rstd_in[row];
      const float k = dot[r] * rstd * rstd / (float)dim;
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int c = (j * NT + threadIdx.x) * V;
        Vec16<T> o;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float gf = to_f(gv[r][j].v[i]), xf = to_f(xv[r][j].v[i]);
          o.v[i] = from_f<T>(rstd * (gf * wf[j][i] - xf * k));
          acc[j][i] += gf * xf * rstd;
        }
        if (c < dim) st16(dx + (size_t)row * dim + c, o);
      }
    }
  }
  float* out = dw_partial + (size_t)blockIdx.x * dim;
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = (j * NT + threadIdx.x) * V;
    if (c < dim) {
#pragma unroll
      for (int i = 0; i < V; ++i) out[c + i] = acc[j][i];
    }
  }
}

// ---- dispatch -------------------------------------------------------------------------------------------------
// Rows of up to 8 * 8 * 32 vectors (16384 elements of 16 bits) stay in registers.
template <typename T>
__host__ inline bool fwd_fast(const T* x, const T* w, T* y, float* rstd, int rows, int dim, float eps,
                              cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  const int lanes_vecs = (dim / V + 31) / 32;  // vectors per lane if one warp held the row
#define TB_RMS_FWD(CH, WPR)                                                                                   \
  fwd_rowreg_kernel<T, CH, WPR><<<(rows + (8 / WPR) - 1) / (8 / WPR), 256, 0, st>>>(x, w, y, rstd, rows, dim, eps)
  if (lanes_vecs <= 1) TB_RMS_FWD(1, 1);
  else if (lanes_vecs <= 2) TB_RMS_FWD(2, 1);
  else if (lanes_vecs <= 4) TB_RMS_FWD(4, 1);
  else if (lanes_vecs <= 8) TB_RMS_FWD(4, 2);
  else if (lanes_vecs <= 16) TB_RMS_FWD(4, 4);
  else if (lanes_vecs <= 32) TB_RMS_FWD(4, 8);
  else if (lanes_vecs <= 64) TB_RMS_FWD(8, 8);
  else return false;
#undef TB_RMS_FWD
  return true;
}

struct BwdPlan {
  int variant;  // 0 = warp per row, 1 = CTA per row group
  int nt, ch, r;
  int grid;
};

// `cap` bounds the grid (= number of partial rows the caller's scratch can hold).
__host__ inline BwdPlan bwd_plan(int rows, int dim, int vec, int cap) {
  BwdPlan p{};
  const int vecs = dim / vec;  // 16-byte vectors per row
  if (vecs <= 64) {            // <= 2 vectors per lane (4 would need 178 registers: one CTA per SM)
    p.variant = 0;
    p.ch = vecs <= 32 ? 1 : 2;
    p.grid = (rows + 8 * 4 - 1) / (8 * 4);  // about four rows per warp
    const int full = 148 * 8;
    if (p.grid > full) p.grid = full;
  } else {
    p.variant = 1;
    p.nt = vecs <= 256 ? 256 : 512;
    p.ch = (vecs + p.nt - 1) / p.nt;  // 1, 2 or 4 (dim <= 16384 elements of 16 bits)
    if (p.ch == 3) p.ch = 4;
    p.r = p.ch == 1 ? 2 : 1;
    p.grid = (rows + p.r - 1) / p.r;
    const int full = 148 * (p.nt == 256 ? 8 : 4);
    if (p.grid > full) p.grid = full;
  }
  if (p.grid > cap) p.grid = cap;
  if (p.grid < 1) p.grid = 1;
  return p;
}

template <typename T>
__host__ inline bool bwd_fast(const BwdPlan& p, const T* g, const T* x, const T* w, const float* rstd, T* dx,
                              float* part, int rows, int dim, cudaStream_t st) {
#define TB_RMS_ARGS g, x, w, rstd, dx, part, rows, dim
  if (p.variant == 0) {
    if (p.ch == 1) bwd_warp_kernel<T, 1><<<p.grid, 256, 0, st>>>(TB_RMS_ARGS);
    else if (p.ch == 2) bwd_warp_kernel<T, 2><<<p.grid, 256, 0, st>>>(TB_RMS_ARGS);
    else bwd_warp_kernel<T, 4><<<p.grid, 256, 0, st>>>(TB_RMS_ARGS);
    return true;
  }
  if (p.nt == 256 && p.ch == 1) bwd_cta_kernel<T, 256, 1, 2><<<p.grid, 256, 0, st>>>(TB_RMS_ARGS);
  else if (p.nt == 512 && p.ch == 1) bwd_cta_kernel<T, 512, 1, 2><<<p.grid, 512, 0, st>>>(TB_RMS_ARGS);
  else if (p.nt == 512 && p.ch == 2) bwd_cta_kernel<T, 512, 2, 1><<<p.grid, 512, 0, st>>>(TB_RMS_ARGS);
  else if (p.nt == 512 && p.ch == 4) bwd_cta_kernel<T, 512, 4, 1><<<p.grid, 512, 0, st>>>(TB_RMS_ARGS);
  else return false;
#undef TB_RMS_ARGS
  return true;
}
}  // namespace tb_rms
