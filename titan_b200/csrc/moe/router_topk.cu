// MoE router for sm_100a: scores, (biased) top-k choice, gate values, per-expert histogram — one kernel.
//
//   scores = sigmoid(l) | softmax(l) | sqrt(softplus(l))          (fp32, one warp per token, E <= 256)
//   choice = top-k of (scores + bias)        (bias steers the choice only; ties → lowest expert id)
//            or the caller's `forced_idx` (hash routing: expert ids looked up from the token id)
//   gate   = scores[choice]; optionally gate /= Σ gate + 1e-20; gate *= route_scale
//   counts[e] += 1 for every chosen (token, expert) pair                       (integer atomics: exact)
//
// Semantics: the reference's router (models/deepseek_v4/moe.py:125-187: score functions, bias for
// choice, renormalisation and scale, `histc` counts, hash table `tid2eid[vocab, k]`).
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int MAX_PER_LANE = 8;  // E <= 256

__device__ __forceinline__ float softplus_stable(float x) { return x > 20.f ? x : log1pf(__expf(fminf(x, 20.f))); }

__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits,
                                                          const float* __restrict__ bias,
                                                          const long long* __restrict__ forced_idx,
                                                          float* __restrict__ gate, long long* __restrict__ idx_out,
                                                          int* __restrict__ counts, float* __restrict__ scores_out,
                                                          int T, int E, int k, int score_func, int route_norm,
                                                          float route_scale, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int token = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (token >= T) return;
  const float* l = logits + (long long)token * E;
  float s[MAX_PER_LANE];
  // lane owns experts lane, lane+32, ...
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    s[j] = e < E ? l[e] : -INFINITY;
    mx = fmaxf(mx, s[j]);
  }
  if (score_func == 1) {  // softmax
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      s[j] = e < E ? __expf(s[j] - mx) : 0.f;
      sum += s[j];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) s[j] *= inv;
  } else {
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < E) s[j] = score_func == 0 ? 1.f / (1.f + __expf(-s[j])) : sqrtf(softplus_stable(s[j]));
      else s[j] = 0.f;
    }
  }
  if (scores_out != nullptr) {
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < E) scores_out[(long long)token * E + e] = s[j];
    }
  }
  float c[MAX_PER_LANE];  // choice keys
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    c[j] = e < E ? s[j] + (bias != nullptr ? bias[e] : 0.f) : -INFINITY;
  }
  float gsum = 0.f;
  float my_gate = 0.f;  // lane i (< k) keeps the i-th gate
  int my_idx = 0;
  for (int i = 0; i < k; ++i) {
    int best_e;
    if (forced_idx != nullptr) {
      const long long fe = forced_idx[(long long)token * k + i];
      if (fe < 0 || fe >= E) {
        if (lane == 0 && status != nullptr) atomicExch(status, TB_ERR_BOUNDS);
        best_e = 0;
      } else {
        best_e = (int)fe;
      }
    } else {
      float bv = -INFINITY;
      int be = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < MAX_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        if (e < E && (c[j] > bv || (c[j] == bv && e < be))) { bv = c[j]; be = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
      }
      best_e = be;
#pragma unroll
      for (int j = 0; j < MAX_PER_LANE; ++j)
        if (lane + 32 * j == best_e) c[j] = -INFINITY;  // taken
    }
    // fetch the unbiased score of the chosen expert from its owner lane
    float sv = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j)
      if (lane + 32 * j == best_e) sv = s[j];
    sv = __shfl_sync(0xffffffffu, sv, best_e & 31);
    gsum += sv;
    if (lane == i) { my_gate = sv; my_idx = best_e; }
    if (lane == 0 && counts != nullptr) atomicAdd(counts + best_e, 1);
  }
  if (lane < k) {
    float g = my_gate;
    if (route_norm) g = g / (gsum + 1e-20f);
    gate[(long long)token * k + lane] = g * route_scale;
    idx_out[(long long)token * k + lane] = my_idx;
  }
}
}  // namespace

// score_func: 0 sigmoid, 1 softmax, 2 sqrt-softplus.  counts (int32 [E]) is accumulated into (zero it first).
// scores_out (optional, [T, E]) receives the full score matrix for the backward pass.
TB_API int tb_router_topk(const float* logits, const float* bias, const long long* forced_idx, float* gate,
                          long long* idx, int* counts, float* scores_out, int T, int E, int k, int score_func,
                          int route_norm, float route_scale, int* status, cudaStream_t st) {
  if (E < 1 || E > 32 * MAX_PER_LANE || k < 1 || k > 32 || k > E) return TB_ERR_ARG;
  if (T == 0) return 0;
  const int grid = (T + 7) / 8;
  router_topk_kernel<<<grid, 256, 0, st>>>(logits, bias, forced_idx, gate, idx, counts, scores_out, T, E, k,
                                           score_func, route_norm, route_scale, status);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
