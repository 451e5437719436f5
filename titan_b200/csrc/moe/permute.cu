// MoE token permutation into the padded expert-major layout, and its inverse (sm_100a, memory-bound).
//
// Layout: expert e owns rows [start[e], start[e] + count[e]) of the buffer; start[e] is a multiple of
// 128 and the tail up to start[e+1] is zero, so grouped-GEMM tiles never straddle experts and the
// weight-gradient contraction may run over whole tiles.  `offs[e]` = start[e+1] (cumulative padded ends).
// The order of rows inside an expert is the order of the (token, slot) pairs: stable, hence reproducible.
//
//   tb_moe_plan      pair → destination row (`dest[P]`), `offs[E]`, `counts[E]`        (3 small kernels)
//   tb_moe_gather    buf[dest[p]] = x[p / k] * (scale[p] | 1); pad rows zeroed          (dispatch / combine-bwd)
//   tb_moe_combine   out[t] = base[t] + Σ_j buf[dest[t*k+j]] * (w[t*k+j] | 1)           (combine / dispatch-bwd)
//   tb_moe_pair_dot  d[p] = <buf[dest[p]], g[p / k]>                                    (gradient of the weights)
//
// `expert_base` lets a dispatching rank add the rows other ranks place before its own inside every
// expert segment (expert parallelism); with nullptr the plan is local.
//
// Reference ops: `npu_moe_token_permute / _unpermute`, `npu_moe_re_routing`
// (converters/kernels/permutation.py:13-143, moe_dispatch.py:74-107).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int PLAN_THREADS = 256;
constexpr int PAIRS_PER_BLOCK = 1024;  // 32 chunks of 32 pairs
constexpr int MAX_E = 256;
constexpr int ALIGN = 128;

// Row buffers of every expert-parallel rank (index = owner rank; a single entry without EP).  A destination
// code d addresses row (d % capacity) of owner (d / capacity).
struct MoeBufs {
  void* p[8];
};

// pass 1: per-block histogram
__global__ void __launch_bounds__(PLAN_THREADS) plan_hist_kernel(const long long* __restrict__ idx, int P, int E,
                                                                 int* __restrict__ block_counts) {
  __shared__ int h[MAX_E];
  for (int e = threadIdx.x; e < E; e += PLAN_THREADS) h[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * PAIRS_PER_BLOCK;
  for (int i = threadIdx.x; i < PAIRS_PER_BLOCK; i += PLAN_THREADS) {
    const int p = base + i;
    if (p < P) {
      const long long e = idx[p];
      if (e >= 0 && e < E) atomicAdd(&h[(int)e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += PLAN_THREADS) block_counts[blockIdx.x * E + e] = h[e];
}

// pass 2 (one block): exclusive scan over blocks per expert, padded segment starts
__global__ void __launch_bounds__(MAX_E) plan_scan_kernel(int* __restrict__ block_counts, int nblocks, int E,
                                                          const int* __restrict__ expert_base,
                                                          const int* __restrict__ expert_total,
                                                          int* __restrict__ counts, int* __restrict__ starts,
                                                          int* __restrict__ offs, int capacity,
                                                          int experts_per_owner, int* __restrict__ status) {
  __shared__ int tot[MAX_E];
  const int e = threadIdx.x;
  if (e < E) {
    int run = expert_base != nullptr ? expert_base[e] : 0;  // rows of lower ranks come first
    int mine = 0;
    for (int b = 0; b < nblocks; ++b) {
      const int c = block_counts[b * E + e];
      block_counts[b * E + e] = run;
      run += c;
      mine += c;
    }
    counts[e] = mine;
    tot[e] = expert_total != nullptr ? expert_total[e] : mine;  // rows of all ranks in this expert's segment
  }
  __syncthreads();
  if (e == 0) {
    // with expert parallelism every owner rank has its own buffer: row numbering restarts per owner
    int acc = 0, worst = 0;
    for (int i = 0; i < E; ++i) {
      if (experts_per_owner > 0 && i % experts_per_owner == 0) acc = 0;
      starts[i] = acc;
      acc += (tot[i] + ALIGN - 1) / ALIGN * ALIGN;
      offs[i] = acc;
      worst = max(worst, acc);
    }
    if (worst > capacity && status != nullptr) atomicExch(status, TB_ERR_BOUNDS);
  }
}

// pass 3: stable destination of every pair
__global__ void __launch_bounds__(PLAN_THREADS) plan_assign_kernel(const long long* __restrict__ idx, int P, int E,
                                                                   const int* __restrict__ block_base,
                                                                   const int* __restrict__ starts,
                                                                   int* __restrict__ dest, int capacity,
                                                                   int experts_per_owner) {
  extern __shared__ int chunk_cnt[];  // [32 chunks][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * E; i += PLAN_THREADS) chunk_cnt[i] = 0;
  __syncthreads();
  const int base = blockIdx.x * PAIRS_PER_BLOCK;
  int my_e[4], my_rank[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int chunk = warp * 4 + r;
    const int p = base + chunk * 32 + lane;
    long long e = p < P ? idx[p] : -1;
    if (e < 0 || e >= E) e = -1;
    my_e[r] = (int)e;
    const unsigned same = __match_any_sync(0xffffffffu, my_e[r]);
    my_rank[r] = __popc(same & ((1u << lane) - 1u));
    if (my_e[r] >= 0 && my_rank[r] == 0) chunk_cnt[chunk * E + my_e[r]] = __popc(same);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += PLAN_THREADS) {  // exclusive scan over the 32 chunks
    int run = 0;
    for (int c = 0; c < 32; ++c) {
      const int v = chunk_cnt[c * E + e];
      chunk_cnt[c * E + e] = run;
      run += v;
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int chunk = warp * 4 + r;
    const int p = base + chunk * 32 + lane;
    if (p >= P) continue;
    int d = -1;
    if (my_e[r] >= 0) {
      d = starts[my_e[r]] + block_base[blockIdx.x * E + my_e[r]] + chunk_cnt[chunk * E + my_e[r]] + my_rank[r];
      if (d >= capacity) d = -1;  // over capacity: the pair is dropped (status already raised by the scan)
      else if (experts_per_owner > 0) d += (my_e[r] / experts_per_owner) * capacity;  // owner-major encoding
    }
    dest[p] = d;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gather_kernel(const T* __restrict__ x, const int* __restrict__ dest,
                                                     const float* __restrict__ scale, MoeBufs bufs, int nown, int P,
                                                     int k, int dim, long long buf_rows) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long p = warp0; p < P; p += nwarps) {
    const int d = dest[p];
    if (d < 0 || d >= buf_rows * nown) continue;
    const T* src = x + (p / k) * dim;
    T* dst = reinterpret_cast<T*>(bufs.p[d / buf_rows]) + (long long)(d % buf_rows) * dim;
    const float sc = scale != nullptr ? scale[p] : 1.f;
    for (int c = lane * V; c < dim; c += 32 * V) {
      Vec16<T> v = ld16(src + c);
      if (scale != nullptr) {
#pragma unroll
        for (int i = 0; i < V; ++i) v.v[i] = from_f<T>(to_f(v.v[i]) * sc);
      }
      st16(dst + c, v);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) zero_pad_kernel(T* __restrict__ buf, const int* __restrict__ starts,
                                                       const int* __restrict__ totals, const int* __restrict__ offs,
                                                       int dim, long long buf_rows) {
  constexpr int V = Vec16<T>::N;
  const int e = blockIdx.x;
  const int r0 = starts[e] + totals[e], r1 = offs[e];
  Vec16<T> z;
#pragma unroll
  for (int i = 0; i < V; ++i) z.v[i] = from_f<T>(0.f);
  const long long n = (long long)(r1 - r0) * (dim / V);
  for (long long i = threadIdx.x; i < n; i += blockDim.x) {
    const long long row = r0 + i / (dim / V);
    if (row < buf_rows) st16(buf + row * dim + (i % (dim / V)) * V, z);
  }
}

// dst[row] = src[row] for the rows an expert received, 0 for its alignment padding; rows past the last expert's end
// are not touched (nobody reads them).  One pass over the USED part of a capacity-sized buffer: the copy out of (or
// into) a staging buffer and the padding fill in one launch, independent of the capacity factor.
template <typename T>
__global__ void __launch_bounds__(256) take_kernel(const T* __restrict__ src, T* __restrict__ dst,
                                                   const int* __restrict__ starts, const int* __restrict__ totals,
                                                   const int* __restrict__ offs, int dim, long long buf_rows) {
  constexpr int V = Vec16<T>::N;
  const int e = blockIdx.y;
  const int r_begin = e > 0 ? offs[e - 1] : 0, r_end = offs[e];
  const int v_begin = starts[e], v_end = starts[e] + totals[e];
  const int per_row = dim / V;
  Vec16<T> z;
#pragma unroll
  for (int i = 0; i < V; ++i) z.v[i] = from_f<T>(0.f);
  const long long n = (long long)(r_end - r_begin) * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long row = r_begin + i / per_row;
    if (row >= buf_rows) continue;
    const long long o = row * dim + (i % per_row) * V;
    st16(dst + o, (row >= v_begin && row < v_end) ? ld16(src + o) : z);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) combine_kernel(MoeBufs bufs, int nown, const int* __restrict__ dest,
                                                      const float* __restrict__ w, const T* __restrict__ base,
                                                      T* __restrict__ out, int Tn, int k, int dim,
                                                      long long buf_rows) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  constexpr int KMAX = 8;   // slots whose row pointers and weights are kept in registers (top-k of every model here)
  for (long long t = warp0; t < Tn; t += nwarps) {
    if (k <= KMAX) {
      // the k expert rows of this token: resolve the indices once, then issue all row loads of a column chunk
      // back to back before the first use (the slot order of the sum stays fixed: reproducible)
      const T* rows[KMAX];
      float ws[KMAX];
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        rows[j] = nullptr;
        ws[j] = 0.f;
        if (j < k) {
          const int d = dest[t * k + j];
          if (d >= 0 && d < buf_rows * nown) {
            rows[j] = reinterpret_cast<const T*>(bufs.p[d / buf_rows]) + (long long)(d % buf_rows) * dim;
            ws[j] = w != nullptr ? w[t * k + j] : 1.f;
          }
        }
      }
      for (int c = lane * V; c < dim; c += 32 * V) {
        Vec16<T> v[KMAX];
#pragma unroll
        for (int j = 0; j < KMAX; ++j)
          if (rows[j] != nullptr) v[j] = ld16(rows[j] + c);
        float acc[V];
        if (base != nullptr) {
          const Vec16<T> b = ld16(base + t * dim + c);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] = to_f(b.v[i]);
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < KMAX; ++j)
          if (rows[j] != nullptr) {
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] += to_f(v[j].v[i]) * ws[j];
          }
        Vec16<T> o;
#pragma unroll
        for (int i = 0; i < V; ++i) o.v[i] = from_f<T>(acc[i]);
        st16(out + t * dim + c, o);
      }
      continue;
    }
    for (int c = lane * V; c < dim; c += 32 * V) {
      float acc[V];
      if (base != nullptr) {
        const Vec16<T> b = ld16(base + t * dim + c);
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = to_f(b.v[i]);
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = 0.f;
      }
      for (int j = 0; j < k; ++j) {  // fixed slot order: reproducible sums
        const int d = dest[t * k + j];
        if (d < 0 || d >= buf_rows * nown) continue;
        const float wj = w != nullptr ? w[t * k + j] : 1.f;
        const Vec16<T> v = ld16(reinterpret_cast<const T*>(bufs.p[d / buf_rows]) + (long long)(d % buf_rows) * dim + c);
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] += to_f(v.v[i]) * wj;
      }
      Vec16<T> o;
#pragma unroll
      for (int i = 0; i < V; ++i) o.v[i] = from_f<T>(acc[i]);
      st16(out + t * dim + c, o);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) pair_dot_kernel(MoeBufs bufs, int nown, const int* __restrict__ dest,
                                                       const T* __restrict__ g, float* __restrict__ d, int P, int k,
                                                       int dim, long long buf_rows) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long p = warp0; p < P; p += nwarps) {
    const int r = dest[p];
    float acc = 0.f;
    if (r >= 0 && r < buf_rows * nown) {
      const T* row = reinterpret_cast<const T*>(bufs.p[r / buf_rows]) + (long long)(r % buf_rows) * dim;
      for (int c = lane * V; c < dim; c += 32 * V) {
        const Vec16<T> a = ld16(row + c), b = ld16(g + (p / k) * dim + c);
#pragma unroll
        for (int i = 0; i < V; ++i) acc += to_f(a.v[i]) * to_f(b.v[i]);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) d[p] = acc;
  }
}

int rows_grid(long long rows) {
  long long g = (rows + 7) / 8;
  if (g > 148LL * 8) g = 148LL * 8;
  return g < 1 ? 1 : (int)g;
}
}  // namespace

TB_API int tb_moe_plan_blocks(int P) { return (P + PAIRS_PER_BLOCK - 1) / PAIRS_PER_BLOCK; }

// idx: [P] expert id per (token, slot) pair (int64; out-of-range ids are dropped).
// scratch: tb_moe_plan_blocks(P) * E int32.  Outputs: dest[P], counts[E] (this rank's rows per expert),
// starts[E], offs[E].  expert_base / expert_total (optional, [E]): rows that precede this rank's rows inside
// each expert segment and the segment's total over all ranks (expert parallelism).
TB_API int tb_moe_plan(const long long* idx, int P, int E, const int* expert_base, const int* expert_total,
                       int* scratch, int* dest, int* counts, int* starts, int* offs, int capacity,
                       int experts_per_owner, int* status, cudaStream_t st) {
  if (E < 1 || E > MAX_E || P < 0) return TB_ERR_ARG;
  const int nb = tb_moe_plan_blocks(P);
  if (nb > 0) {
    plan_hist_kernel<<<nb, PLAN_THREADS, 0, st>>>(idx, P, E, scratch);
    TB_CUDA_CHECK(cudaGetLastError());
  }
  plan_scan_kernel<<<1, MAX_E, 0, st>>>(scratch, nb, E, expert_base, expert_total, counts, starts, offs, capacity,
                                        experts_per_owner, status);
  TB_CUDA_CHECK(cudaGetLastError());
  if (nb > 0) {
    plan_assign_kernel<<<nb, PLAN_THREADS, 32 * E * sizeof(int), st>>>(idx, P, E, scratch, starts, dest, capacity,
                                                                       experts_per_owner);
    TB_CUDA_CHECK(cudaGetLastError());
  }
  tb_note_launch(nb > 0 ? 3 : 1);
  return 0;
}

#define TB_MOE_DT(dtype, ...)                                  \
  switch (dtype) {                                             \
    case 0: { using T = float; __VA_ARGS__; break; }           \
    case 1: { using T = __nv_bfloat16; __VA_ARGS__; break; }   \
    case 2: { using T = __half; __VA_ARGS__; break; }          \
    default: return TB_ERR_ARG;                                \
  }

static int fill_bufs(MoeBufs& b, void* const* ptrs, int nown) {
  if (nown < 1 || nown > 8) return TB_ERR_ARG;
  for (int i = 0; i < 8; ++i) b.p[i] = i < nown ? ptrs[i] : nullptr;
  return 0;
}

// bufs[owner][row] = x[p / k] * scale[p] for dest[p] = owner * buf_rows + row (peer stores when owner is remote).
TB_API int tb_moe_gather(const void* x, const int* dest, const float* scale, void* const* bufs, int nown, int P, int k,
                         int dim, long long buf_rows, int dtype, cudaStream_t st) {
  MoeBufs b;
  if (int rc = fill_bufs(b, bufs, nown)) return rc;
  if (P == 0) return 0;
  TB_MOE_DT(dtype, {
    if (dim % Vec16<T>::N) return TB_ERR_ARG;
    gather_kernel<T><<<rows_grid(P), 256, 0, st>>>((const T*)x, dest, scale, b, nown, P, k, dim, buf_rows);
  });
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

// Zero the alignment padding [starts[e] + totals[e], offs[e]) of experts e in [0, E) of a local buffer.
TB_API int tb_moe_zero_pad(void* buf, const int* starts, const int* totals, const int* offs, int E, int dim,
                           long long buf_rows, int dtype, cudaStream_t st) {
  if (E <= 0) return 0;
  TB_MOE_DT(dtype, {
    if (dim % Vec16<T>::N) return TB_ERR_ARG;
    zero_pad_kernel<T><<<E, 256, 0, st>>>((T*)buf, starts, totals, offs, dim, buf_rows);
  });
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

// Copy the received rows of experts e in [0, E) from `src` to `dst` (both [buf_rows, dim]) and zero their alignment
// padding [starts[e] + totals[e], offs[e]); see take_kernel.
TB_API int tb_moe_take(const void* src, void* dst, const int* starts, const int* totals, const int* offs, int E,
                       int dim, long long buf_rows, int dtype, cudaStream_t st) {
  if (E <= 0) return 0;
  TB_MOE_DT(dtype, {
    if (dim % Vec16<T>::N) return TB_ERR_ARG;
    take_kernel<T><<<dim3(148 * 2 / (E < 148 ? E : 148) + 1, E), 256, 0, st>>>((const T*)src, (T*)dst, starts, totals,
                                                                              offs, dim, buf_rows);
  });
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

TB_API int tb_moe_combine(void* const* bufs, int nown, const int* dest, const float* w, const void* base, void* out,
                          int Tn, int k, int dim, long long buf_rows, int dtype, cudaStream_t st) {
  MoeBufs b;
  if (int rc = fill_bufs(b, bufs, nown)) return rc;
  if (Tn == 0) return 0;
  TB_MOE_DT(dtype, {
    if (dim % Vec16<T>::N) return TB_ERR_ARG;
    combine_kernel<T><<<rows_grid(Tn), 256, 0, st>>>(b, nown, dest, w, (const T*)base, (T*)out, Tn, k, dim, buf_rows);
  });
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

TB_API int tb_moe_pair_dot(void* const* bufs, int nown, const int* dest, const void* g, float* d, int P, int k,
                           int dim, long long buf_rows, int dtype, cudaStream_t st) {
  MoeBufs b;
  if (int rc = fill_bufs(b, bufs, nown)) return rc;
  if (P == 0) return 0;
  TB_MOE_DT(dtype, {
    if (dim % Vec16<T>::N) return TB_ERR_ARG;
    pair_dot_kernel<T><<<rows_grid(P), 256, 0, st>>>(b, nown, dest, (const T*)g, d, P, k, dim, buf_rows);
  });
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
