// Multi-tensor fused AdamW / Adam for sm_100a: one launch updates up to TB_ADAM_MAX_TENSORS tensors.
//
//   g' = g * grad_scale                     (grad_scale: optional device scalar = clip coefficient,
//                                            so gradient clipping costs no extra pass over memory)
//   decoupled (AdamW):  p -= lr * wd * p ; m, v EMA of g' ; p -= lr/bc1 * m / (sqrt(v)/sqrt(bc2) + eps)
//   coupled   (Adam) :  g' += wd * p first
//   amsgrad (optional): vmax = max(vmax, v) used in the denominator
//
// Parameters and gradients may be fp32 / bf16 / fp16; the moments are fp32 or bf16.  All math is fp32.
// Work is cut into chunks of TB_ADAM_CHUNK elements; block b handles (tensor[block_tensor[b]],
// chunk block_chunk[b]); the table travels in the kernel parameters, so there is no metadata
// allocation and no host-device sync.
//
// Replaces the per-parameter `torch._fused_adamw_` launches of the reference's optimizers
// (patches/optimizer/swap_optimizer.py:574-591).
#include "../common/tb_common.cuh"

#define TB_ADAM_MAX_TENSORS 24
// 592 = 148 SMs x 4 resident blocks of 512 threads: one balanced wave per launch (480 blocks left 3 or 4 per SM,
// i.e. a fifth of the machine idle while the fuller SMs finished)
#define TB_ADAM_MAX_BLOCKS 592
#define TB_ADAM_CHUNK 65536

struct TbAdamArgs {
  void* p[TB_ADAM_MAX_TENSORS];
  const void* g[TB_ADAM_MAX_TENSORS];
  void* m[TB_ADAM_MAX_TENSORS];
  void* v[TB_ADAM_MAX_TENSORS];
  void* vmax[TB_ADAM_MAX_TENSORS];  // amsgrad only
  long long n[TB_ADAM_MAX_TENSORS];
  unsigned short block_chunk[TB_ADAM_MAX_BLOCKS];  // chunk index inside the slot's window (see `base`)
  unsigned char block_tensor[TB_ADAM_MAX_BLOCKS];
  long long base[TB_ADAM_MAX_TENSORS];             // first element of the slot's window inside its tensor
};

namespace {
using namespace tb;

// 4 consecutive elements as one 16-byte (fp32) or 8-byte (16-bit types) access; `ptr` must be so aligned
__device__ __forceinline__ void load4(const float* ptr, float (&o)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(ptr);
  o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* ptr, float (&o)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(ptr);
  const float2 a = unpack_bf16x2(t.x), b = unpack_bf16x2(t.y);
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}
__device__ __forceinline__ void load4(const __half* ptr, float (&o)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(ptr);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}
__device__ __forceinline__ void store4(float* ptr, const float (&o)[4]) {
  *reinterpret_cast<float4*>(ptr) = make_float4(o[0], o[1], o[2], o[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* ptr, const float (&o)[4]) {
  *reinterpret_cast<uint2*>(ptr) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
}
__device__ __forceinline__ void store4(__half* ptr, const float (&o)[4]) {
  __half2 a = __floats2half2_rn(o[0], o[1]), b = __floats2half2_rn(o[2], o[3]);
  *reinterpret_cast<uint2*>(ptr) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}

template <typename PT, typename GT, typename ST>
__global__ void __launch_bounds__(512) adamw_kernel(const __grid_constant__ TbAdamArgs a, float lr, float beta1,
                                                    float beta2, float eps, float wd, float bc1, float rsqrt_bc2,
                                                    const float* __restrict__ grad_scale,
                                                    const float* __restrict__ dyn, int decoupled, int amsgrad,
                                                    int maximize) {
  // A launch recorded in a CUDA graph reads what changes from step to step (learning rate, bias corrections) from
  // device memory instead of its baked-in arguments.
  if (dyn != nullptr) { lr = dyn[0]; bc1 = dyn[1]; rsqrt_bc2 = dyn[2]; }
  const int t = a.block_tensor[blockIdx.x];
  const long long start = a.base[t] + (long long)a.block_chunk[blockIdx.x] * TB_ADAM_CHUNK;
  const long long n = a.n[t];
  PT* p = (PT*)a.p[t];
  const GT* g = (const GT*)a.g[t];
  ST* m = (ST*)a.m[t];
  ST* v = (ST*)a.v[t];
  ST* vm = (ST*)a.vmax[t];
  float gs = grad_scale != nullptr ? *grad_scale : 1.f;
  if (maximize) gs = -gs;
  const float step_size = lr / bc1;
  const long long end = (start + TB_ADAM_CHUNK < n) ? start + TB_ADAM_CHUNK : n;
  // 4 elements per thread per iteration; tensors from the caching allocator are ≥16B aligned, but shards
  // may start anywhere inside a flat buffer, so vector access is only used when all pointers allow it.
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                        reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                        reinterpret_cast<uintptr_t>(vm)) & 15) == 0;
  auto update = [&](float& pf, float gf, float& mf, float& vf, float& vmf) {
    gf *= gs;
    if (decoupled) pf -= lr * wd * pf; else gf += wd * pf;
    mf = beta1 * mf + (1.f - beta1) * gf;
    vf = beta2 * vf + (1.f - beta2) * gf * gf;
    float denom_v = vf;
    if (amsgrad) { vmf = fmaxf(vmf, vf); denom_v = vmf; }
    pf -= step_size * mf / (sqrtf(denom_v) * rsqrt_bc2 + eps);
  };
  if (vec_ok) {
    auto tail = [&](long long i) {  // fewer than 4 elements left for this thread
      for (long long j = i; j < end; ++j) {
        float pf = to_f(p[j]), mf = to_f(m[j]), vf = to_f(v[j]), xf = amsgrad ? to_f(vm[j]) : 0.f;
        update(pf, to_f(g[j]), mf, vf, xf);
        p[j] = from_f<PT>(pf); m[j] = from_f<ST>(mf); v[j] = from_f<ST>(vf);
        if (amsgrad) vm[j] = from_f<ST>(xf);
      }
    };
    // two groups of 4 elements per thread and iteration: all eight loads are issued before the first update
    for (long long i = start + (long long)threadIdx.x * 4; i < end; i += 512 * 8) {
      const long long j = i + 512 * 4;
      const bool has_a = i + 4 <= end, has_b = j + 4 <= end;
      float pa[4], ga[4], ma[4], va[4], xa[4] = {0, 0, 0, 0};
      float pb[4], gb[4], mb[4], vb[4], xb[4] = {0, 0, 0, 0};
      if (has_a) { load4(p + i, pa); load4(g + i, ga); load4(m + i, ma); load4(v + i, va); if (amsgrad) load4(vm + i, xa); }
      if (has_b) { load4(p + j, pb); load4(g + j, gb); load4(m + j, mb); load4(v + j, vb); if (amsgrad) load4(vm + j, xb); }
      if (has_a) {
#pragma unroll
        for (int k = 0; k < 4; ++k) update(pa[k], ga[k], ma[k], va[k], xa[k]);
        store4(p + i, pa); store4(m + i, ma); store4(v + i, va);
        if (amsgrad) store4(vm + i, xa);
      } else {
        tail(i);
      }
      if (has_b) {
#pragma unroll
        for (int k = 0; k < 4; ++k) update(pb[k], gb[k], mb[k], vb[k], xb[k]);
        store4(p + j, pb); store4(m + j, mb); store4(v + j, vb);
        if (amsgrad) store4(vm + j, xb);
      } else if (j < end) {
        tail(j);
      }
    }
  } else {
    for (long long j = start + threadIdx.x; j < end; j += 512) {
      float pf = to_f(p[j]), mf = to_f(m[j]), vf = to_f(v[j]), xf = amsgrad ? to_f(vm[j]) : 0.f;
      update(pf, to_f(g[j]), mf, vf, xf);
      p[j] = from_f<PT>(pf); m[j] = from_f<ST>(mf); v[j] = from_f<ST>(vf);
      if (amsgrad) vm[j] = from_f<ST>(xf);
    }
  }
}

template <typename PT, typename GT, typename ST>
int launch(const TbAdamArgs& a, int nblocks, float lr, float b1, float b2, float eps, float wd, float bc1,
           float rsqrt_bc2, const float* gs, const float* dyn, int decoupled, int amsgrad, int maximize,
           cudaStream_t st) {
  adamw_kernel<PT, GT, ST><<<nblocks, 512, 0, st>>>(a, lr, b1, b2, eps, wd, bc1, rsqrt_bc2, gs, dyn, decoupled,
                                                    amsgrad, maximize);
  TB_CUDA_CHECK(cudaGetLastError());
  tb_note_launch(1);
  return 0;
}
}  // namespace

TB_API int tb_adam_limits(int* max_tensors, int* max_blocks, int* chunk) {
  *max_tensors = TB_ADAM_MAX_TENSORS;
  *max_blocks = TB_ADAM_MAX_BLOCKS;
  *chunk = TB_ADAM_CHUNK;
  return 0;
}

// Host entry: arrays of `count` tensors (any count; launches are split as needed).
// p_dtype / g_dtype: 0 fp32, 1 bf16, 2 fp16;  s_dtype (moments): 0 fp32, 1 bf16.  step >= 1.
static int adamw_multi_impl(void* const* p, const void* const* g, void* const* m, void* const* v, void* const* vmax,
                            const long long* numel, int count, float lr, float beta1, float beta2, float eps, float wd,
                            long long step, const float* grad_scale, const float* dyn, int decoupled, int amsgrad,
                            int maximize, int p_dtype, int g_dtype, int s_dtype, cudaStream_t st) {
  if (step < 1 || count < 0) return TB_ERR_ARG;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2 = 1.f - powf(beta2, (float)step);
  const float rsqrt_bc2 = 1.f / sqrtf(bc2);
  TbAdamArgs a;
  int nt = 0, nb = 0;
  auto flush = [&]() -> int {
    if (nb == 0) { nt = 0; return 0; }
    int rc = TB_ERR_ARG;
#define TB_GO(PT, GT, ST) rc = launch<PT, GT, ST>(a, nb, lr, beta1, beta2, eps, wd, bc1, rsqrt_bc2, grad_scale, dyn, decoupled, amsgrad, maximize, st)
    const int key = p_dtype * 100 + g_dtype * 10 + s_dtype;
    switch (key) {
      case 0: TB_GO(float, float, float); break;
      case 110: TB_GO(__nv_bfloat16, __nv_bfloat16, float); break;
      case 100: TB_GO(__nv_bfloat16, float, float); break;
      case 111: TB_GO(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16); break;
      case 10: TB_GO(float, __nv_bfloat16, float); break;
      case 220: TB_GO(__half, __half, float); break;
      default: rc = TB_ERR_ARG;
    }
#undef TB_GO
    nt = 0; nb = 0;
    return rc;
  };
  for (int i = 0; i < count; ++i) {
    const long long n = numel[i];
    if (n <= 0) continue;
    long long chunks = (n + TB_ADAM_CHUNK - 1) / TB_ADAM_CHUNK;
    long long done = 0;
    while (done < chunks) {
      if (nt == TB_ADAM_MAX_TENSORS || nb == TB_ADAM_MAX_BLOCKS) { int rc = flush(); if (rc) return rc; }
      const int slot = nt++;
      a.p[slot] = p[i]; a.g[slot] = g[i]; a.m[slot] = m[i]; a.v[slot] = v[i];
      a.vmax[slot] = (amsgrad && vmax != nullptr) ? vmax[i] : nullptr;
      a.n[slot] = n;
      a.base[slot] = done * TB_ADAM_CHUNK;  // a tensor that spans several launches continues where it stopped
      unsigned short local = 0;
      while (done < chunks && nb < TB_ADAM_MAX_BLOCKS) {
        a.block_tensor[nb] = (unsigned char)slot;
        a.block_chunk[nb] = local++;
        ++nb; ++done;
      }
    }
  }
  return flush();
}

TB_API int tb_adamw_multi(void* const* p, const void* const* g, void* const* m, void* const* v, void* const* vmax,
                          const long long* numel, int count, float lr, float beta1, float beta2, float eps, float wd,
                          long long step, const float* grad_scale, int decoupled, int amsgrad, int maximize,
                          int p_dtype, int g_dtype, int s_dtype, cudaStream_t st) {
  return adamw_multi_impl(p, g, m, v, vmax, numel, count, lr, beta1, beta2, eps, wd, step, grad_scale, nullptr,
                          decoupled, amsgrad, maximize, p_dtype, g_dtype, s_dtype, st);
}

// The bias corrections exactly as tb_adamw_multi computes them on the host (fp32): out = {1 - beta1^step,
// 1 / sqrt(1 - beta2^step)}.  The graph form fills its device buffer from these, so both forms agree bit for bit.
TB_API int tb_adamw_bias_corrections(float beta1, float beta2, long long step, float* out) {
  if (step < 1 || out == nullptr) return TB_ERR_ARG;
  out[0] = 1.f - powf(beta1, (float)step);
  out[1] = 1.f / sqrtf(1.f - powf(beta2, (float)step));
  return 0;
}

// The same update with the per-step scalars read from device memory: `dyn` = {lr, 1 - beta1^step,
// 1 / sqrt(1 - beta2^step)}.  For launches recorded in a CUDA graph, which are replayed with new scalars every step.
TB_API int tb_adamw_multi_dyn(void* const* p, const void* const* g, void* const* m, void* const* v, void* const* vmax,
                              const long long* numel, int count, const float* dyn, float beta1, float beta2, float eps,
                              float wd, const float* grad_scale, int decoupled, int amsgrad, int maximize, int p_dtype,
                              int g_dtype, int s_dtype, cudaStream_t st) {
  if (dyn == nullptr) return TB_ERR_ARG;
  return adamw_multi_impl(p, g, m, v, vmax, numel, count, 0.f, beta1, beta2, eps, wd, 1, grad_scale, dyn, decoupled,
                          amsgrad, maximize, p_dtype, g_dtype, s_dtype, st);
}

// ---------------------------------------------------------------------------------------------------------------
// Multi-tensor sum of squares (the gradient norm before clipping): block b reduces one chunk of one tensor and writes
// ONE partial; the caller sums the partials (a fixed order, so the norm is reproducible).  Same chunk table as AdamW.
struct TbSumSqArgs {
  const void* g[TB_ADAM_MAX_TENSORS];
  long long n[TB_ADAM_MAX_TENSORS];
  long long base[TB_ADAM_MAX_TENSORS];
  unsigned short block_chunk[TB_ADAM_MAX_BLOCKS];
  unsigned char block_tensor[TB_ADAM_MAX_BLOCKS];
};

namespace {
template <typename GT>
__global__ void __launch_bounds__(512) sumsq_kernel(const __grid_constant__ TbSumSqArgs a, float* __restrict__ out) {
  const int t = a.block_tensor[blockIdx.x];
  const long long start = a.base[t] + (long long)a.block_chunk[blockIdx.x] * TB_ADAM_CHUNK;
  const long long n = a.n[t];
  const GT* g = (const GT*)a.g[t];
  const long long end = (start + TB_ADAM_CHUNK < n) ? start + TB_ADAM_CHUNK : n;
  float acc0 = 0.f, acc1 = 0.f;
  if ((reinterpret_cast<uintptr_t>(g) & 15) == 0) {
    constexpr int V = tb::Vec16<GT>::N;
    long long i = start + (long long)threadIdx.x * V;
    for (; i + V <= end; i += 512LL * V) {
      const tb::Vec16<GT> v = tb::ld16(g + i);
#pragma unroll
      for (int k = 0; k < V; k += 2) {
        const float x = tb::to_f(v.v[k]), y = tb::to_f(v.v[k + 1]);
        acc0 = fmaf(x, x, acc0); acc1 = fmaf(y, y, acc1);
      }
    }
    if (i < end) {  // at most one thread holds the ragged tail of the chunk
      for (long long j = i; j < end && j < i + V; ++j) { const float x = tb::to_f(g[j]); acc0 = fmaf(x, x, acc0); }
    }
  } else {
    for (long long j = start + threadIdx.x; j < end; j += 512) { const float x = tb::to_f(g[j]); acc0 = fmaf(x, x, acc0); }
  }
  float s = tb::warp_sum(acc0 + acc1);
  __shared__ float part[16];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < 16 ? part[threadIdx.x] : 0.f;
    s = tb::warp_sum(s);
    if (threadIdx.x == 0) out[blockIdx.x] = s;
  }
}
}  // namespace

// partials: float[capacity]; on return *written partials hold Σ g² of consecutive chunks.  dtype: 0 fp32, 1 bf16, 2 fp16.
TB_API int tb_multi_sumsq(const void* const* g, const long long* numel, int count, int dtype, float* partials,
                          long long capacity, long long* written, cudaStream_t st) {
  if (count < 0 || (dtype != 0 && dtype != 1 && dtype != 2)) return TB_ERR_ARG;
  TbSumSqArgs a;
  int nt = 0, nb = 0;
  long long out_pos = 0;
  auto flush = [&]() -> int {
    if (nb == 0) { nt = 0; return 0; }
    if (out_pos + nb > capacity) return TB_ERR_ARG;
    float* out = partials + out_pos;
    if (dtype == 0) sumsq_kernel<float><<<nb, 512, 0, st>>>(a, out);
    else if (dtype == 1) sumsq_kernel<__nv_bfloat16><<<nb, 512, 0, st>>>(a, out);
    else sumsq_kernel<__half><<<nb, 512, 0, st>>>(a, out);
    TB_CUDA_CHECK(cudaGetLastError());
    tb_note_launch(1);
    out_pos += nb;
    nt = 0; nb = 0;
    return 0;
  };
  for (int i = 0; i < count; ++i) {
    const long long n = numel[i];
    if (n <= 0) continue;
    const long long chunks = (n + TB_ADAM_CHUNK - 1) / TB_ADAM_CHUNK;
    long long done = 0;
    while (done < chunks) {
      if (nt == TB_ADAM_MAX_TENSORS || nb == TB_ADAM_MAX_BLOCKS) { if (int rc = flush()) return rc; }
      const int slot = nt++;
      a.g[slot] = g[i]; a.n[slot] = n; a.base[slot] = done * TB_ADAM_CHUNK;
      unsigned short local = 0;
      while (done < chunks && nb < TB_ADAM_MAX_BLOCKS) {
        a.block_tensor[nb] = (unsigned char)slot;
        a.block_chunk[nb] = local++;
        ++nb; ++done;
      }
    }
  }
  if (int rc = flush()) return rc;
  *written = out_pos;
  return 0;
}
