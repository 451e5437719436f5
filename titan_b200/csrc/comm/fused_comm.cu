// Compute fused with collectives over NVLink peer memory (plain P2P loads / stores; no multicast).
//
//   tb_ag_gemm            C = gather_rows(A_shards) · B      A tiles are TMA-loaded from the owner GPU
//   tb_ag_b_gemm          C = A · gather_rows(B_shards)ᵀ     weight shards gathered inside the GEMM (FSDP)
//   tb_gemm_rs            partial C tiles are stored into the owner's staging slot, flags released
//   tb_rs_reduce          owner sums the nranks staged partials once every source's flag has arrived
//   tb_castscale_rs       gradient bucket reduce-scatter: read chunk `rank` of every peer's bucket,
//                         sum in fp32, scale, cast — one pass, no intermediate buffers
//   tb_signal / tb_wait_flags / tb_barrier_all   flag plumbing with time-bounded waits
//
// Flags are 32-bit epoch counters in symmetric memory: a waiter compares `flag - epoch >= 0` so the
// counters may wrap.  Peers' buffers are reached through pointers exchanged by the host (CUDA VMM
// handles); every wait gives up after ~2 s and records TB_ERR_WAIT_PEER in the status word.
//
// Counterparts in the reference: `npu_all_gather_base_mm`, `npu_mm_reduce_scatter_base`
// (patches/torch/micro_pipeline_tp.py:35-105) and the FSDP2 all-gather / reduce-scatter it inherits.
#include <cstdlib>

#include "../gemm/gemm_kernel.cuh"

using namespace tbg;

namespace {

struct PeerPtrs {
  void* p[MAX_RANKS];
};

// How many CTAs copy instead of multiply: a copier keeps about 190 KB in flight, i.e. roughly 40 GB/s of a link with a
// few microseconds of latency, so a link-bound problem wants dozens of them and a compute-bound one few.  The share of
// SMs follows the share of the link in (link time + GEMM time), between 8 and 40.
int pick_copiers(double flops, double link_bytes, int nranks) {
  if (nranks <= 1) return 0;
  if (const char* env = getenv("TITAN_B200_COPIERS")) {  // tuning knob: fixed number of copier CTAs
    const int c = atoi(env);
    if (c >= 1 && c <= 64) return c;
  }
  const double t_gemm = flops / 1.4e15, t_link = link_bytes / 7.0e11;
  int c = (int)(148.0 * t_link / (t_link + t_gemm) * 0.6);
  return c < 8 ? 8 : (c > 40 ? 40 : c);
}

__global__ void signal_kernel(PeerPtrs flags, int slot, unsigned int value, int nranks) {
  const int r = threadIdx.x;
  if (r < nranks) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned int*>(flags.p[r]) + slot, value);
  }
}

__global__ void wait_flags_kernel(const unsigned int* flags, int first, int count, unsigned int value, int* status) {
  const int i = threadIdx.x;
  if (i < count) {
    if (!wait_flag_ge(flags + first + i, value, nullptr) && status != nullptr) atomicExch(status, TB_ERR_WAIT_PEER);
  }
}

// out[i] = scale * Σ_src in_src[rank_chunk + i]
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(512) castscale_rs_kernel(PeerPtrs in, TOut* __restrict__ out, long long chunk,
                                                           long long chunk_offset, int nranks, int rank, float scale) {
  constexpr int V = Vec16<TIn>::N;
  const long long nvec = chunk / V;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = 0.f;
    for (int s = 0; s < nranks; ++s) {
      const int src = (rank + s) % nranks;  // start with the local bucket; peers in ring order
      const Vec16<TIn> v = ld16(reinterpret_cast<const TIn*>(in.p[src]) + chunk_offset + i * V);
#pragma unroll
      for (int k = 0; k < V; ++k) acc[k] += to_f(v.v[k]);
    }
#pragma unroll
    for (int k = 0; k < V; ++k) out[i * V + k] = from_f<TOut>(acc[k] * scale);
  }
  for (long long i = nvec * V + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < chunk;
       i += (long long)gridDim.x * blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < nranks; ++s)
      a += to_f(reinterpret_cast<const TIn*>(in.p[(rank + s) % nranks])[chunk_offset + i]);
    out[i] = from_f<TOut>(a * scale);
  }
}

// The same reduction done INSIDE the NVSwitch: `mc` is the multicast address of the symmetric slot (all ranks'
// buckets bound to one multicast object), and one `multimem.ld_reduce` returns the sum over the ranks of 16 bytes,
// accumulated in fp32 for bf16 data.  Each rank asks for its own chunk only, so every byte crosses its link once.
template <typename TOut>
__global__ void __launch_bounds__(512) castscale_rs_nvls_bf16_kernel(const __nv_bfloat16* __restrict__ mc,
                                                                      TOut* __restrict__ out, long long chunk,
                                                                      float scale) {
  const long long nvec = chunk / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    uint32_t r0, r1, r2, r3;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "l"(mc + i * 8)
                 : "memory");
    const uint32_t r[4] = {r0, r1, r2, r3};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16x2(r[k]);
      out[i * 8 + 2 * k] = from_f<TOut>(f.x * scale);
      out[i * 8 + 2 * k + 1] = from_f<TOut>(f.y * scale);
    }
  }
}

template <typename TOut>
__global__ void __launch_bounds__(512) castscale_rs_nvls_f32_kernel(const float* __restrict__ mc, TOut* __restrict__ out,
                                                                     long long chunk, float scale) {
  const long long nvec = chunk / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float a, b, c, d;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(a), "=f"(b), "=f"(c), "=f"(d)
                 : "l"(mc + i * 4)
                 : "memory");
    out[i * 4] = from_f<TOut>(a * scale);
    out[i * 4 + 1] = from_f<TOut>(b * scale);
    out[i * 4 + 2] = from_f<TOut>(c * scale);
    out[i * 4 + 3] = from_f<TOut>(d * scale);
  }
}

// out[row, :] = Σ_src stage[src][row, :]; each block first makes sure all sources have published
template <typename T>
__global__ void __launch_bounds__(256) rs_reduce_kernel(const T* __restrict__ stage, const unsigned int* flags,
                                                        unsigned int epoch, T* __restrict__ out, long long numel,
                                                        int nranks, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < nranks) {
    if (!wait_flag_ge(flags + threadIdx.x, epoch, nullptr)) {
      ok = 0;
      if (status != nullptr) atomicExch(status, TB_ERR_WAIT_PEER);
    }
  }
  __syncthreads();
  if (!ok) return;
  constexpr int V = Vec16<T>::N;
  const long long nvec = numel / V;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = 0.f;
    for (int s = 0; s < nranks; ++s) {
      const Vec16<T> v = ld16(stage + (long long)s * numel + i * V);
#pragma unroll
      for (int k = 0; k < V; ++k) acc[k] += to_f(v.v[k]);
    }
    Vec16<T> o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.v[k] = from_f<T>(acc[k]);
    st16(out + i * V, o);
  }
}

}  // namespace

// Write `value` into slot `slot` of the flag array of every rank (flag_ptrs[r] = that rank's array).
TB_API int tb_signal(void* const* flag_ptrs, int nranks, int slot, unsigned int value, cudaStream_t st) {
  if (nranks < 1 || nranks > MAX_RANKS) return TB_ERR_ARG;
  PeerPtrs f{};
  for (int r = 0; r < nranks; ++r) f.p[r] = flag_ptrs[r];
  signal_kernel<<<1, 32, 0, st>>>(f, slot, value, nranks);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

// Wait until local flags[first .. first+count) have all reached `value` (bounded; reports through `status`).
TB_API int tb_wait_flags(const unsigned int* flags, int first, int count, unsigned int value, int* status,
                         cudaStream_t st) {
  if (count < 1 || count > 32) return TB_ERR_ARG;
  wait_flags_kernel<<<1, 32, 0, st>>>(flags, first, count, value, status);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

// C[M,N] = concat_r(A_r)[M,K] · B[N,K]ᵀ where A_r = a_ptrs[r] is rank r's [m_shard, K] shard (K-major).
// ready_flags: local array, slot r is set to >= epoch by rank r once its shard may be read.
// gathered: local [M, K] buffer that receives the remote shards (each crosses NVLink exactly once; the rows of
// this rank's own shard are not written).  chunk_flags: local zero-initialised uint32 [2 * M / 128] (flags, then piece counters), reused across
// calls with increasing epochs.
TB_API int tb_ag_gemm(void* const* a_ptrs, const void* B, void* C, void* gathered, unsigned int* chunk_flags, int M,
                      int N, int K, int m_shard, int b_mn, int dtype, int rank, int nranks,
                      const unsigned int* ready_flags, unsigned int epoch, int* status, cudaStream_t st) {
  if (nranks < 1 || nranks > MAX_RANKS || m_shard % BM || m_shard * nranks != M) return TB_ERR_ARG;
  if ((K % 8) || (N % 8) || (dtype != 1 && dtype != 2)) return TB_ERR_ARG;
  AMaps am;
  CUtensorMap tb_;
  CMaps cm;
  if (int rc = make_a_map(&am.m[0], a_ptrs[rank], dtype, 0, (uint64_t)m_shard, (uint64_t)K, K)) return rc;
  if (int rc = make_a_map(&am.m[1], gathered, dtype, 0, (uint64_t)M, (uint64_t)K, K)) return rc;
  if (int rc = make_b_map(&tb_, B, dtype, b_mn, (uint64_t)N, (uint64_t)K, b_mn ? N : K)) return rc;
  if (int rc = make_c_map(&cm.m[0], C, dtype, (uint64_t)M, (uint64_t)N, N)) return rc;
  GemmParams p{};
  p.mode = ALLGATHER; p.M = M; p.N = N; p.K = K; p.a_mn = 0; p.b_mn = b_mn; p.is_bf16 = dtype == 1;
  p.ldc = N; p.C = C; p.status = status; p.rank = rank; p.nranks = nranks; p.m_shard = m_shard;
  p.ready_flags = ready_flags; p.epoch = epoch; p.tma_store = 1;
  for (int r = 0; r < nranks; ++r) p.peer_src[r] = a_ptrs[r];
  p.gather_dst = gathered; p.chunk_flags = chunk_flags;
  p.num_copiers = pick_copiers(2.0 * M * N * K, (double)(nranks - 1) * m_shard * K * 2, nranks);
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  int workers = sm_count() - p.num_copiers;
  if (tiles < workers) workers = tiles;
  // copiers and GEMM CTAs wait on one another: all of them must be resident, i.e. the grid fits the SMs
  return launch(am, tb_, cm, p, workers + p.num_copiers, st);
}

// C[M,N] = A[M,K] · concat_r(B_r)[N,K]ᵀ where B_r = b_ptrs[r] is rank r's [n_shard, K] weight shard.
// gathered: local [N, K] buffer for the remote weight shards; chunk_flags: local uint32 [2 * N / 256] (flags, then piece counters).
TB_API int tb_ag_b_gemm(const void* A, void* const* b_ptrs, void* C, void* gathered, unsigned int* chunk_flags, int M,
                        int N, int K, int n_shard, int dtype, int rank, int nranks,
                        const unsigned int* ready_flags, unsigned int epoch, int* status, cudaStream_t st) {
  if (nranks < 1 || nranks > MAX_RANKS || n_shard % BN || n_shard * nranks != N) return TB_ERR_ARG;
  if ((K % 8) || (dtype != 1 && dtype != 2)) return TB_ERR_ARG;
  AMaps am;
  CUtensorMap ta;
  CMaps cm;
  if (int rc = make_b_map(&am.m[0], b_ptrs[rank], dtype, 0, (uint64_t)n_shard, (uint64_t)K, K)) return rc;
  if (int rc = make_b_map(&am.m[1], gathered, dtype, 0, (uint64_t)N, (uint64_t)K, K)) return rc;
  if (int rc = make_a_map(&ta, A, dtype, 0, (uint64_t)M, (uint64_t)K, K)) return rc;
  if (int rc = make_c_map(&cm.m[0], C, dtype, (uint64_t)M, (uint64_t)N, N)) return rc;
  GemmParams p{};
  p.mode = ALLGATHER_B; p.M = M; p.N = N; p.K = K; p.is_bf16 = dtype == 1;
  p.ldc = N; p.C = C; p.status = status; p.rank = rank; p.nranks = nranks; p.n_shard = n_shard;
  p.ready_flags = ready_flags; p.epoch = epoch; p.tma_store = 1;
  for (int r = 0; r < nranks; ++r) p.peer_src[r] = b_ptrs[r];
  p.gather_dst = gathered; p.chunk_flags = chunk_flags;
  // every output tile group walks all weight chunks, so the whole gather sits in front of the GEMM: at least 16
  // copiers (measured on 2 GPUs, 8192x28672x4096: 1.68 ms with 8, 1.54 with 16, 1.61 with 24, 1.75 with 36)
  p.num_copiers = pick_copiers(2.0 * M * N * K, (double)(nranks - 1) * n_shard * K * 2, nranks);
  if (nranks > 1 && p.num_copiers < 16 && getenv("TITAN_B200_COPIERS") == nullptr) p.num_copiers = 16;
  const int tiles = ((M + BM - 1) / BM) * (N / BN);
  int workers = sm_count() - p.num_copiers;
  if (tiles < workers) workers = tiles;
  return launch(am, ta, cm, p, workers + p.num_copiers, st);
}

// Partial product of this rank, scattered by rows: rows of owner d go to stage_ptrs[d] + [rank][m_shard][N].
// peer_flags[d] + rank is released with `epoch` once all of this rank's tiles for d are stored.
TB_API int tb_gemm_rs(const void* A, const void* B, void* const* stage_ptrs, void* const* peer_flags,
                      unsigned int* tile_counters, int M, int N, int K, int m_shard, int b_mn, int dtype, int rank,
                      int nranks, unsigned int epoch, int* status, cudaStream_t st) {
  if (nranks < 1 || nranks > MAX_RANKS || m_shard % BM || m_shard * nranks != M) return TB_ERR_ARG;
  if ((K % 8) || (N % 8) || (dtype != 1 && dtype != 2)) return TB_ERR_ARG;
  AMaps am;
  CUtensorMap tb_;
  if (int rc = make_a_map(&am.m[0], A, dtype, 0, (uint64_t)M, (uint64_t)K, K)) return rc;
  if (int rc = make_b_map(&tb_, B, dtype, b_mn, (uint64_t)N, (uint64_t)K, b_mn ? N : K)) return rc;
  GemmParams p{};
  p.mode = SCATTER; p.M = M; p.N = N; p.K = K; p.b_mn = b_mn; p.is_bf16 = dtype == 1;
  p.ldc = N; p.C = nullptr; p.status = status; p.rank = rank; p.nranks = nranks; p.m_shard = m_shard;
  p.epoch = epoch; p.tile_counters = tile_counters;
  CMaps cm;
  for (int r = 0; r < nranks; ++r) {
    p.stage_ptrs[r] = stage_ptrs[r];
    p.peer_flags[r] = reinterpret_cast<unsigned int*>(peer_flags[r]);
    // every owner's staging area [nranks * m_shard, N]: whole tiles go there as bulk tensor stores
    if (int rc = make_c_map(&cm.m[r], stage_ptrs[r], dtype, (uint64_t)nranks * m_shard, (uint64_t)N, N)) return rc;
  }
  p.tma_store = 1;
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  return launch(am, tb_, cm, p, tiles < sm_count() ? tiles : sm_count(), st);
}

// out[m_shard, N] = Σ_src stage[src]; waits (bounded) for flags[0..nranks) >= epoch first.
TB_API int tb_rs_reduce(const void* stage, const unsigned int* flags, unsigned int epoch, void* out, long long numel,
                        int nranks, int dtype, int* status, cudaStream_t st) {
  if (nranks < 1 || nranks > MAX_RANKS || numel <= 0) return TB_ERR_ARG;
  long long grid = (numel / 8 + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  if (grid < 1) grid = 1;
  if (dtype == 1)
    rs_reduce_kernel<__nv_bfloat16><<<(int)grid, 256, 0, st>>>((const __nv_bfloat16*)stage, flags, epoch,
                                                               (__nv_bfloat16*)out, numel, nranks, status);
  else if (dtype == 2)
    rs_reduce_kernel<__half><<<(int)grid, 256, 0, st>>>((const __half*)stage, flags, epoch, (__half*)out, numel,
                                                        nranks, status);
  else
    return TB_ERR_ARG;
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

// Gradient reduce-scatter with cast and scale.  in_ptrs[r]: rank r's full bucket (numel = chunk * nranks);
// out: this rank's chunk.  in_dtype: 0 fp32 / 1 bf16; out_dtype: 0 fp32 / 1 bf16.  Callers order this after
// a flag exchange that says every bucket is complete.
TB_API int tb_castscale_rs(void* const* in_ptrs, void* out, long long chunk, int rank, int nranks, float scale,
                           int in_dtype, int out_dtype, cudaStream_t st) {
  if (nranks < 1 || nranks > MAX_RANKS || chunk <= 0) return TB_ERR_ARG;
  PeerPtrs in{};
  for (int r = 0; r < nranks; ++r) in.p[r] = in_ptrs[r];
  long long grid = (chunk / 8 + 511) / 512;
  if (grid > 148 * 4) grid = 148 * 4;
  if (grid < 1) grid = 1;
  const long long off = chunk * rank;
  if ((off * (in_dtype == 0 ? 4 : 2)) % 16 != 0) return TB_ERR_ARG;
#define TB_RS(TI, TO) castscale_rs_kernel<TI, TO><<<(int)grid, 512, 0, st>>>(in, (TO*)out, chunk, off, nranks, rank, scale)
  if (in_dtype == 1 && out_dtype == 0) TB_RS(__nv_bfloat16, float);
  else if (in_dtype == 1 && out_dtype == 1) TB_RS(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == 0 && out_dtype == 0) TB_RS(float, float);
  else if (in_dtype == 0 && out_dtype == 1) TB_RS(float, __nv_bfloat16);
  else return TB_ERR_ARG;
#undef TB_RS
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

// In-switch variant of tb_castscale_rs: `mc_chunk` is the MULTICAST address of this rank's chunk inside the symmetric
// slot (multicast base + the slot's offset + rank * chunk elements); `chunk` elements, a multiple of 8 (bf16) or 4
// (fp32), 16-byte aligned.  Callers order it after the same flag exchange.
TB_API int tb_castscale_rs_nvls(const void* mc_chunk, void* out, long long chunk, float scale, int in_dtype,
                                int out_dtype, cudaStream_t st) {
  if (mc_chunk == nullptr || chunk <= 0 || (reinterpret_cast<uintptr_t>(mc_chunk) & 15) != 0) return TB_ERR_ARG;
  if (chunk % (in_dtype == 1 ? 8 : 4) != 0) return TB_ERR_ARG;
  long long grid = (chunk / 8 + 511) / 512;
  if (grid > 148 * 4) grid = 148 * 4;
  if (grid < 1) grid = 1;
  if (in_dtype == 1 && out_dtype == 0)
    castscale_rs_nvls_bf16_kernel<float><<<(int)grid, 512, 0, st>>>((const __nv_bfloat16*)mc_chunk, (float*)out, chunk, scale);
  else if (in_dtype == 1 && out_dtype == 1)
    castscale_rs_nvls_bf16_kernel<__nv_bfloat16><<<(int)grid, 512, 0, st>>>((const __nv_bfloat16*)mc_chunk, (__nv_bfloat16*)out, chunk, scale);
  else if (in_dtype == 0 && out_dtype == 0)
    castscale_rs_nvls_f32_kernel<float><<<(int)grid, 512, 0, st>>>((const float*)mc_chunk, (float*)out, chunk, scale);
  else if (in_dtype == 0 && out_dtype == 1)
    castscale_rs_nvls_f32_kernel<__nv_bfloat16><<<(int)grid, 512, 0, st>>>((const float*)mc_chunk, (__nv_bfloat16*)out, chunk, scale);
  else return TB_ERR_ARG;
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

namespace {
__global__ void put_kernel(PeerPtrs dst, const unsigned int* __restrict__ src, long long nwords, int nranks) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nwords;
       i += (long long)gridDim.x * blockDim.x) {
    const unsigned int v = src[i];
    for (int r = 0; r < nranks; ++r) reinterpret_cast<unsigned int*>(dst.p[r])[i] = v;
  }
}
}  // namespace

// Copy `nbytes` (multiple of 4) from local `src` to dst_ptrs[r] on every rank (small control data: counts, sizes).
TB_API int tb_put(void* const* dst_ptrs, int nranks, const void* src, long long nbytes, cudaStream_t st) {
  if (nranks < 1 || nranks > MAX_RANKS || nbytes % 4) return TB_ERR_ARG;
  if (nbytes == 0) return 0;
  PeerPtrs d{};
  for (int r = 0; r < nranks; ++r) d.p[r] = dst_ptrs[r];
  long long grid = (nbytes / 4 + 255) / 256;
  if (grid > 64) grid = 64;
  put_kernel<<<(int)grid, 256, 0, st>>>(d, (const unsigned int*)src, nbytes / 4, nranks);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Ulysses context parallelism: the head <-> sequence all-to-all fused into the projections on either side of it
// (reference: distributed/context_parallel/ulysses_cp.py:28-64 does chunk -> all_to_all -> cat around the attention).
//
// tb_gemm_a2a_scatter: C = A[M,K] · B[N,K]ᵀ (or B[K,N] with b_mn) where M = batch * seq_local rows of this rank's
// sequence slice and the N columns are heads; columns [r*n_shard, (r+1)*n_shard) are stored into rank r's receive
// buffer recv_ptrs[r] = [batch * seq_local * nranks, n_shard] at rows b*seq_full + rank*seq_local + s.
// peer_flags[r] + rank is released with `epoch` when all of this rank's boxes for r have landed.
TB_API int tb_gemm_a2a_scatter(const void* A, const void* B, void* const* recv_ptrs, void* const* peer_flags,
                               unsigned int* tile_counters, int M, int N, int K, int n_shard, int seq_local, int b_mn,
                               int dtype, int rank, int nranks, unsigned int epoch, int* status, cudaStream_t st) {
  if (nranks < 1 || nranks > MAX_RANKS || n_shard % 64 || n_shard * nranks != N) return TB_ERR_ARG;
  if (seq_local <= 0 || seq_local % BM || M % seq_local || (K % 8) || (dtype != 1 && dtype != 2)) return TB_ERR_ARG;
  AMaps am;
  CUtensorMap tb_;
  CMaps cm;
  if (int rc = make_a_map(&am.m[0], A, dtype, 0, (uint64_t)M, (uint64_t)K, K)) return rc;
  if (int rc = make_b_map(&tb_, B, dtype, b_mn, (uint64_t)N, (uint64_t)K, b_mn ? N : K)) return rc;
  GemmParams p{};
  p.mode = SCATTER_N; p.M = M; p.N = N; p.K = K; p.b_mn = b_mn; p.is_bf16 = dtype == 1;
  p.ldc = N; p.C = nullptr; p.status = status; p.rank = rank; p.nranks = nranks; p.n_shard = n_shard;
  p.seq_local = seq_local; p.seq_full = seq_local * nranks;
  p.epoch = epoch; p.tile_counters = tile_counters; p.tma_store = 1;
  for (int r = 0; r < nranks; ++r) {
    p.peer_flags[r] = reinterpret_cast<unsigned int*>(peer_flags[r]);
    if (int rc = make_c_map(&cm.m[r], recv_ptrs[r], dtype, (uint64_t)M * nranks, (uint64_t)n_shard, n_shard))
      return rc;
  }
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  return launch(am, tb_, cm, p, tiles < sm_count() ? tiles : sm_count(), st);
}

// tb_a2a_gather_gemm: C[M,N] = gather_k(A)[M, nranks*k_shard] · B[N,K]ᵀ (or B[K,N] with b_mn).  Rank r holds the
// k_shard columns [r*k_shard, ...) of every rank's rows in a_ptrs[r] = [batch * seq_full, k_shard]; this rank's rows
// are b*seq_full + rank*seq_local + s.  gathered: local [nranks, M, k_shard] buffer (the remote slices land there,
// each crossing NVLink once); chunk_flags: local uint32 [2 * nranks * M / 128] (flags, then piece counters).
TB_API int tb_a2a_gather_gemm(void* const* a_ptrs, const void* B, void* C, void* gathered, unsigned int* chunk_flags,
                              int M, int N, int k_shard, int seq_local, int b_mn, int dtype, int rank, int nranks,
                              const unsigned int* ready_flags, unsigned int epoch, int* status, cudaStream_t st) {
  if (nranks < 1 || nranks > MAX_RANKS || k_shard <= 0 || k_shard % BK) return TB_ERR_ARG;
  if (seq_local <= 0 || seq_local % BM || M % seq_local || (N % 8) || (dtype != 1 && dtype != 2)) return TB_ERR_ARG;
  const int K = k_shard * nranks;
  AMaps am;
  CUtensorMap tb_;
  CMaps cm;
  if (int rc = make_a_map(&am.m[0], a_ptrs[rank], dtype, 0, (uint64_t)M * nranks, (uint64_t)k_shard, k_shard))
    return rc;
  if (int rc = make_a_map(&am.m[1], gathered, dtype, 0, (uint64_t)M * nranks, (uint64_t)k_shard, k_shard)) return rc;
  if (int rc = make_b_map(&tb_, B, dtype, b_mn, (uint64_t)N, (uint64_t)K, b_mn ? N : K)) return rc;
  if (int rc = make_c_map(&cm.m[0], C, dtype, (uint64_t)M, (uint64_t)N, N)) return rc;
  GemmParams p{};
  p.mode = GATHER_K; p.M = M; p.N = N; p.K = K; p.b_mn = b_mn; p.is_bf16 = dtype == 1;
  p.ldc = N; p.C = C; p.status = status; p.rank = rank; p.nranks = nranks; p.k_shard = k_shard;
  p.seq_local = seq_local; p.seq_full = seq_local * nranks;
  p.ready_flags = ready_flags; p.epoch = epoch; p.tma_store = 1;
  for (int r = 0; r < nranks; ++r) p.peer_src[r] = a_ptrs[r];
  p.gather_dst = gathered; p.chunk_flags = chunk_flags;
  p.num_copiers = pick_copiers(2.0 * M * N * K, (double)(nranks - 1) * M * k_shard * 2, nranks);
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  int workers = sm_count() - p.num_copiers;
  if (tiles < workers) workers = tiles;
  return launch(am, tb_, cm, p, workers + p.num_copiers, st);
}
