// Row-wise top-k selection over long score rows (lightning indexer: up to 131072 keys, k up to 2048).
//
// One CTA per query row.  Row r may only look at its first (pos_offset + r + 1) / ratio keys (causal prefix; ratio > 1
// for compressed keys that stand for `ratio` tokens each), so masked entries are never read and need not exist.  Selection is an exact radix select on the order-preserving integer
// image of the fp32 scores: four 8-bit histogram rounds find the k-th largest key, a last pass emits every
// element above it plus as many ties as still fit.  The emitted SET is exact; the order inside a row is
// arbitrary (consumers gather by index).  Rows with fewer than k visible keys are padded with index -1 and
// value -inf.
//
// Semantics: `topk` of the masked index scores in the reference (models/deepseek_v32/model.py:363-395), with
// -1 padding as in models/deepseek_v4/model.py:654-656.
#include "../common/tb_common.cuh"

namespace {
using namespace tb;

constexpr int TK_THREADS = 512;

__device__ __forceinline__ uint32_t ordered_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float → larger unsigned
}

__global__ void __launch_bounds__(TK_THREADS) topk_select_kernel(const float* __restrict__ scores, long long ld,
                                                                 int rows, int T, int k, int pos_offset,
                                                                 int ratio, int* __restrict__ out_idx,
                                                                 float* __restrict__ out_val) {
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining, s_count_gt, s_count_eq;
  const int r = blockIdx.x;
  if (r >= rows) return;
  const float* row = scores + (long long)r * ld;
  long long vis = ((long long)pos_offset + r + 1) / ratio;
  const int n = (int)(vis < 0 ? 0 : (vis > T ? T : vis));
  int* oi = out_idx + (long long)r * k;
  float* ov = out_val != nullptr ? out_val + (long long)r * k : nullptr;
  if (n <= k) {  // everything visible is selected
    for (int i = threadIdx.x; i < k; i += TK_THREADS) {
      oi[i] = i < n ? i : -1;
      if (ov) ov[i] = i < n ? row[i] : -INFINITY;
    }
    return;
  }
  if (threadIdx.x == 0) { s_prefix = 0; s_remaining = k; }
  __syncthreads();
  for (int round = 0; round < 4; ++round) {
    for (int i = threadIdx.x; i < 256; i += TK_THREADS) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const int shift = 24 - 8 * round;
    for (int i = threadIdx.x; i < n; i += TK_THREADS) {
      const uint32_t key = ordered_key(row[i]);
      if (round == 0 || (key >> (shift + 8)) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int need = s_remaining, b = 255, above = 0;
      for (; b > 0; --b) {
        if (above + hist[b] >= need) break;
        above += hist[b];
      }
      s_remaining = need - above;  // how many to take from bucket b (and, after the last round, from ties)
      s_prefix = (prefix << 8) | (uint32_t)b;
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;  // key of the k-th largest element
  const int ties_wanted = s_remaining;
  if (threadIdx.x == 0) { s_count_gt = 0; s_count_eq = 0; }
  __syncthreads();
  const int n_gt = k - ties_wanted;
  for (int i = threadIdx.x; i < n; i += TK_THREADS) {
    const float x = row[i];
    const uint32_t key = ordered_key(x);
    int slot = -1;
    if (key > thr) {
      slot = atomicAdd(&s_count_gt, 1);
    } else if (key == thr) {
      const int e = atomicAdd(&s_count_eq, 1);
      if (e < ties_wanted) slot = n_gt + e;
    }
    if (slot >= 0 && slot < k) {
      oi[slot] = i;
      if (ov) ov[slot] = x;
    }
  }
}
}  // namespace

// scores: [rows, ld] fp32; out_idx: [rows, k] int32; out_val: [rows, k] fp32 or nullptr.
TB_API int tb_topk_select(const float* scores, long long ld, int rows, int T, int k, int pos_offset, int ratio,
                          int* out_idx, float* out_val, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (k < 1 || T < 1 || ratio < 1) return TB_ERR_ARG;
  topk_select_kernel<<<rows, TK_THREADS, 0, st>>>(scores, ld, rows, T, k, pos_offset, ratio, out_idx, out_val);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
