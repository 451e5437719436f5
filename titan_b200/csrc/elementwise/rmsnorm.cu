// RMSNorm forward / backward for sm_100a (memory-bound; one warp per row, 16-byte accesses).
//
//   y = x * rsqrt(mean(x^2) + eps) * w            (statistics in fp32; rstd is returned for backward)
//   dx = rstd * (g*w - x * rstd^2 * mean(g*w*x))
//   dw = sum_rows g * x * rstd
//
// Backward accumulates dw per warp in shared memory (each lane owns its columns, no atomics, fixed
// summation order), writes one partial row per CTA into a scratch buffer `dw_partial[grid, dim]`
// and a second kernel reduces the partials in a fixed order: results are bitwise reproducible.
//
// Semantics follow the reference's fused norm op (converters/kernels/rms_norm.py:39-44:
// `npu_rms_norm(x, w, eps)` returning (y, rstd)).
#include "../common/tb_common.cuh"
#include "rmsnorm_fast.cuh"

namespace {

using namespace tb;

template <typename T>
__global__ void __launch_bounds__(128) rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                          T* __restrict__ y, float* __restrict__ rstd_out, int rows,
                                                          int dim, float eps) {
  constexpr int V = Vec16<T>::N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + warp;
  if (row >= rows) return;
  const T* xr = x + (size_t)row * dim;
  T* yr = y + (size_t)row * dim;
  float ss = 0.f;
  for (int c = lane * V; c < dim; c += 32 * V) {
    Vec16<T> xv = ld16(xr + c);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float f = to_f(xv.v[i]);
      ss += f * f;
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)dim + eps);
  if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
  for (int c = lane * V; c < dim; c += 32 * V) {
    Vec16<T> xv = ld16(xr + c);  // second read hits L1/L2
    Vec16<T> wv = ld16(w + c);
    Vec16<T> o;
#pragma unroll
    for (int i = 0; i < V; ++i) o.v[i] = from_f<T>(to_f(xv.v[i]) * rstd * to_f(wv.v[i]));
    st16(yr + c, o);
  }
}

// dynamic smem: WARPS * dim floats
template <typename T, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) rmsnorm_bwd_kernel(const T* __restrict__ g, const T* __restrict__ x,
                                                                 const T* __restrict__ w,
                                                                 const float* __restrict__ rstd_in,
                                                                 T* __restrict__ dx, float* __restrict__ dw_partial,
                                                                 int rows, int dim) {
  constexpr int V = Vec16<T>::N;
  // [WARPS][dimp], dimp = dim rounded up to 32*V.  Within each chunk of 32*V columns the accumulator of
  // column (lane*V + i) sits at (i*32 + lane): consecutive lanes hit consecutive banks.
  extern __shared__ float acc[];
  const int dimp = (dim + 32 * V - 1) / (32 * V) * (32 * V);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* my = acc + (size_t)warp * dimp;
  for (int c = lane; c < dimp; c += 32) my[c] = 0.f;
  __syncwarp();
  for (int row = blockIdx.x * WARPS + warp; row < rows; row += gridDim.x * WARPS) {
    const T* gr = g + (size_t)row * dim;
    const T* xr = x + (size_t)row * dim;
    T* dr = dx + (size_t)row * dim;
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int c = lane * V; c < dim; c += 32 * V) {
      Vec16<T> gv = ld16(gr + c), xv = ld16(xr + c), wv = ld16(w + c);
#pragma unroll
      for (int i = 0; i < V; ++i) dot += to_f(gv.v[i]) * to_f(wv.v[i]) * to_f(xv.v[i]);
    }
    dot = warp_sum(dot);
    const float k = dot * rstd * rstd / (float)dim;
    for (int c = lane * V; c < dim; c += 32 * V) {
      Vec16<T> gv = ld16(gr + c), xv = ld16(xr + c), wv = ld16(w + c);
      Vec16<T> o;
      float* slot = my + (c - lane * V) + lane;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float gf = to_f(gv.v[i]), xf = to_f(xv.v[i]);
        o.v[i] = from_f<T>(rstd * (gf * to_f(wv.v[i]) - xf * k));
        slot[i * 32] += gf * xf * rstd;
      }
      st16(dr + c, o);
    }
  }
  __syncthreads();
  float* out = dw_partial + (size_t)blockIdx.x * dim;
  for (int j = threadIdx.x; j < dimp; j += WARPS * 32) {
    const int chunk = j / (32 * V), rem = j % (32 * V);
    const int col = chunk * 32 * V + (rem & 31) * V + (rem >> 5);
    if (col >= dim) continue;
    float s = 0.f;
#pragma unroll
    for (int wi = 0; wi < WARPS; ++wi) s += acc[(size_t)wi * dimp + j];
    out[col] = s;
  }
}

template <typename T>
__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, T* __restrict__ dw, int nparts, int dim) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= dim) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[(size_t)p * dim + c];
  dw[c] = from_f<T>(s);
}

template <typename T>
int fwd_impl(const void* x, const void* w, void* y, float* rstd, int rows, int dim, float eps, cudaStream_t st) {
  if (dim % Vec16<T>::N != 0) return TB_ERR_ARG;
  const int grid = (rows + 3) / 4;
  if (grid == 0) return 0;
  if (tb_rms::fwd_fast<T>((const T*)x, (const T*)w, (T*)y, rstd, rows, dim, eps, st)) {
    TB_CUDA_CHECK(cudaGetLastError());
    tb_note_launch(1);
    return 0;
  }
  // rows too long for registers: two passes, the second one from L1/L2
  rmsnorm_fwd_kernel<T><<<grid, 128, 0, st>>>((const T*)x, (const T*)w, (T*)y, rstd, rows, dim, eps);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

template <typename T, int WARPS>
int bwd_launch(const void* g, const void* x, const void* w, const float* rstd, void* dx, void* dw, float* scratch,
               int grid, int rows, int dim, cudaStream_t st) {
  constexpr int CH = 32 * Vec16<T>::N;
  const size_t smem = (size_t)WARPS * ((dim + CH - 1) / CH * CH) * sizeof(float);
  auto kern = rmsnorm_bwd_kernel<T, WARPS>;
  if (smem > 48 * 1024)  // per-device attribute; setting it again is cheap
    TB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, WARPS * 32, smem, st>>>((const T*)g, (const T*)x, (const T*)w, rstd, (T*)dx, scratch, rows, dim);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  rmsnorm_dw_reduce_kernel<T><<<(dim + 255) / 256, 256, 0, st>>>(scratch, (T*)dw, grid, dim);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

}  // namespace

namespace {
int legacy_bwd_grid(int rows, int dim) {
  const int warps = dim <= 8192 ? 4 : 2;
  int grid = (rows + warps - 1) / warps;
  const int cap = 148 * 2;
  if (grid > cap) grid = cap;
  return grid < 1 ? 1 : grid;
}

constexpr int kBwdGridCap = 148 * 8;

// 16-bit types take the register-resident kernels for every supported dim; fp32 rows beyond 8192 elements do not
// fit and keep the shared-memory kernel.
bool bwd_uses_fast(int dim, int vec) { return dim % vec == 0 && (dim / vec + 511) / 512 <= 4; }
}  // namespace

// Number of partial rows the backward writes (= its grid size); scratch must hold grid*dim floats.  The vector
// width only matters for fp32 rows longer than 8192 elements, which report the (larger) bound of both layouts.
TB_API int tb_rmsnorm_bwd_grid(int rows, int dim) {
  const int fast = tb_rms::bwd_plan(rows, dim, 8, kBwdGridCap).grid;
  const int fast32 = tb_rms::bwd_plan(rows, dim, 4, kBwdGridCap).grid;
  const int legacy = legacy_bwd_grid(rows, dim);
  int m = fast > fast32 ? fast : fast32;
  return m > legacy ? m : legacy;
}

// dtype: 0 = fp32, 1 = bf16, 2 = fp16
TB_API int tb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int dim, float eps, int dtype,
                          cudaStream_t st) {
  switch (dtype) {
    case 0: return fwd_impl<float>(x, w, y, rstd, rows, dim, eps, st);
    case 1: return fwd_impl<__nv_bfloat16>(x, w, y, rstd, rows, dim, eps, st);
    case 2: return fwd_impl<__half>(x, w, y, rstd, rows, dim, eps, st);
  }
  return TB_ERR_ARG;
}

// `scratch` holds tb_rmsnorm_bwd_grid(rows, dim) * dim floats; it is fully overwritten.
TB_API int tb_rmsnorm_bwd(const void* g, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                          float* scratch, int rows, int dim, int dtype, cudaStream_t st) {
  if (dim > 16384 || rows < 1) return TB_ERR_ARG;
  const int grid = legacy_bwd_grid(rows, dim);
#define TB_BWD(T)                                                                              \
  do {                                                                                         \
    if (dim % Vec16<T>::N != 0) return TB_ERR_ARG;                                             \
    if (bwd_uses_fast(dim, Vec16<T>::N)) {                                                     \
      const tb_rms::BwdPlan plan = tb_rms::bwd_plan(rows, dim, Vec16<T>::N, kBwdGridCap);      \
      if (tb_rms::bwd_fast<T>(plan, (const T*)g, (const T*)x, (const T*)w, rstd, (T*)dx, scratch, rows, dim, st)) { \
        TB_CUDA_CHECK(cudaGetLastError());                                                     \
        tb_note_launch(1);                                                                     \
        rmsnorm_dw_reduce_kernel<T><<<(dim + 255) / 256, 256, 0, st>>>(scratch, (T*)dw, plan.grid, dim); \
        TB_CUDA_CHECK(cudaGetLastError());                                                     \
        tb_note_launch(1);                                                                     \
        return 0;                                                                              \
      }                                                                                        \
    }                                                                                          \
    if (dim <= 8192) return bwd_launch<T, 4>(g, x, w, rstd, dx, dw, scratch, grid, rows, dim, st); \
    return bwd_launch<T, 2>(g, x, w, rstd, dx, dw, scratch, grid, rows, dim, st);              \
  } while (0)
  switch (dtype) {
    case 0: TB_BWD(float);
    case 1: TB_BWD(__nv_bfloat16);
    case 2: TB_BWD(__half);
  }
#undef TB_BWD
  return TB_ERR_ARG;
}

// ---------------------------------------------------------------------------------------------------------
// Allocation-free variant (declaration and contract: rmsnorm_noalloc.h).
#include "rmsnorm_noalloc.h"

#include <atomic>
#include <mutex>

// Scratch for the per-CTA partial sums of dw.  In host code this name is only a handle for the symbol, not a
// device address: the address is looked up per device with cudaGetSymbolAddress and handed to the kernel.
static __device__ __align__(256) float g_rmsnorm_noalloc_scratch[TB_RMSNORM_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
std::atomic<float*> g_noalloc_scratch_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;  // taken only while a device's address is resolved for the first time

// Device address of the scratch array on the current device.  After the first call per device this is one
// acquire load: no lock on the path of a latency-critical caller.
int noalloc_scratch_for_current_device(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TB_NOALLOC_ERR_SYMBOL;
  float* p = g_noalloc_scratch_ptr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    p = g_noalloc_scratch_ptr[dev].load(std::memory_order_relaxed);
    if (p == nullptr) {
      if (cudaGetSymbolAddress((void**)&p, g_rmsnorm_noalloc_scratch) != cudaSuccess || p == nullptr) {
        (void)cudaGetLastError();
        return TB_NOALLOC_ERR_SYMBOL;
      }
      g_noalloc_scratch_ptr[dev].store(p, std::memory_order_release);
    }
  }
  *out = p;
  return 0;
}

template <typename T>
int noalloc_launch(const void* g, const void* x, const void* w, const float* rstd, void* dx, void* dw, float* scratch,
                   int rows, int dim, cudaStream_t st) {
  if (dim % Vec16<T>::N != 0) return TB_NOALLOC_ERR_SHAPE;
  int grid = (rows + 3) / 4;  // four warps (rows) per CTA
  if (grid > TB_RMSNORM_NOALLOC_MAX_PARTIAL_ROWS) grid = TB_RMSNORM_NOALLOC_MAX_PARTIAL_ROWS;
  // grid * dim <= MAX_PARTIAL_ROWS * MAX_DIM floats: the partial rows always fit the static array
  return bwd_launch<T, 4>(g, x, w, rstd, dx, dw, scratch, grid, rows, dim, st);
}
}  // namespace

extern "C" __attribute__((visibility("default"))) int tb_rmsnorm_bwd_noalloc(const void* g, const void* x,
                                                                             const void* w, const float* rstd,
                                                                             void* dx, void* dw, int rows, int dim,
                                                                             int dtype, cudaStream_t stream) {
  if (dim > TB_RMSNORM_NOALLOC_MAX_DIM) return TB_NOALLOC_ERR_TOO_LARGE;
  if (rows < 1 || dim < 1 || dtype < 0 || dtype > 2) return TB_NOALLOC_ERR_SHAPE;
  float* scratch = nullptr;
  if (int rc = noalloc_scratch_for_current_device(&scratch)) return rc;
  switch (dtype) {
    case 0: return noalloc_launch<float>(g, x, w, rstd, dx, dw, scratch, rows, dim, stream);
    case 1: return noalloc_launch<__nv_bfloat16>(g, x, w, rstd, dx, dw, scratch, rows, dim, stream);
    default: return noalloc_launch<__half>(g, x, w, rstd, dx, dw, scratch, rows, dim, stream);
  }
}

extern "C" __attribute__((visibility("default"))) const char* tb_rmsnorm_bwd_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case TB_NOALLOC_ERR_TOO_LARGE:
      return "dim exceeds TB_RMSNORM_NOALLOC_MAX_DIM (8192): the built-in scratch array cannot hold the partial sums";
    case TB_NOALLOC_ERR_SHAPE:
      return "invalid shape or dtype: rows >= 1, dim a multiple of the 16-byte vector, dtype in {0, 1, 2}";
    case TB_NOALLOC_ERR_SYMBOL:
      return "could not obtain the device address of the built-in scratch array on the current device";
    default:
      return code >= 1000 ? "CUDA runtime error (code - 1000)" : "unknown error";
  }
}
