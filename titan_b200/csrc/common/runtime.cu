// Library-wide runtime bookkeeping: launch counter and version.
#include "tb_common.cuh"

#include <atomic>

namespace {
std::atomic<long long> g_launches{0};
}

// called by every host launcher after a successful <<<>>>
extern "C" __attribute__((visibility("default"))) void tb_note_launch(int n) { g_launches.fetch_add(n); }

// Number of kernels this library has launched in this process (benchmarks report it).
TB_API long long tb_launch_count() { return g_launches.load(); }
TB_API int tb_reset_launch_count() { g_launches.store(0); return 0; }
TB_API int tb_version() { return 1; }

// Make `device` current for the calling thread in this library's CUDA runtime (autograd worker threads
// start without a context; multi-GPU processes must never fall back to device 0).
TB_API int tb_bind_device(int device) {
  TB_CUDA_CHECK(cudaSetDevice(device));
  TB_CUDA_CHECK(cudaFree(nullptr));
  return 0;
}

// One asynchronous device-to-device copy on `st` (copy engine; `src` may be a peer GPU's memory mapped into this
// process).  Collectives that should not occupy SMs (the FSDP parameter all-gather) are built from these.
TB_API int tb_peer_copy(void* dst, const void* src, long long bytes, cudaStream_t st) {
  if (bytes <= 0) return 0;
  TB_CUDA_CHECK(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, st));
  return 0;
}
