/* RMSNorm backward for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference: its fused norm op allocates its own workspace
 * through the framework's allocator.  It exists for hosts that cannot do that, for example
 *   - a process whose device memory is owned entirely by its own arena (an inference server or a
 *     training job that reserved all of HBM up front): a cudaMalloc from a library would fail or fragment
 *     that arena;
 *   - latency-sensitive loops where an allocation call may synchronise the device or take a lock
 *     shared with other threads;
 *   - plug-in code called from a runtime that forbids allocation inside its callbacks.
 *
 * The regular entry point `tb_rmsnorm_bwd` needs a caller-provided scratch buffer for its per-CTA partial
 * sums of dw.  Here that scratch is a fixed array that lives in the library image itself
 * (TB_RMSNORM_NOALLOC_SCRATCH_FLOATS floats = 4 MiB, resident on every GPU that loads the library until the
 * process exits).  The caller passes inputs and outputs only.
 *
 * Limits and rules
 *   - dim <= TB_RMSNORM_NOALLOC_MAX_DIM, dim a multiple of the 16-byte vector (8 for 16-bit types, 4 for
 *     fp32), rows >= 1.  Anything else is rejected with TB_NOALLOC_ERR_TOO_LARGE / TB_NOALLOC_ERR_SHAPE
 *     before any work is queued; `tb_rmsnorm_bwd_noalloc_strerror` turns a code into text.
 *   - The function calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - The first call on each device looks up the device address of the scratch array (once per device, with
 *     that device current, under a lock); every later call reads the cached address without taking any lock.
 *     Make that first call before starting any stream capture.
 *   - The scratch used is the one of the CURRENT device (cudaGetDevice) at the time of the call: `stream` must
 *     belong to that device.  A stream of another device is not detected and would run the kernel against the
 *     wrong device's array.
 *   - All calls on a device share the one array, and it keeps the contents of the previous call.  The kernel
 *     overwrites every partial row it later reads, so nothing needs clearing, but two calls that overlap on
 *     the GPU (different streams, no ordering between them) race on the array: order them.
 *
 * Arguments are those of `tb_rmsnorm_bwd` without the scratch pointer:
 *   g, x   [rows, dim]   upstream gradient and forward input      w [dim]   norm weight
 *   rstd   [rows] fp32   reciprocal RMS saved by the forward      dx [rows, dim], dw [dim]   outputs
 *   dtype  0 = fp32, 1 = bf16, 2 = fp16 (all of g, x, w, dx, dw)
 * Returns 0 on success.
 */
#pragma once

#include <cuda_runtime.h>

#define TB_RMSNORM_NOALLOC_MAX_DIM 8192
#define TB_RMSNORM_NOALLOC_MAX_PARTIAL_ROWS 128
#define TB_RMSNORM_NOALLOC_SCRATCH_FLOATS (TB_RMSNORM_NOALLOC_MAX_PARTIAL_ROWS * TB_RMSNORM_NOALLOC_MAX_DIM)

#define TB_NOALLOC_ERR_TOO_LARGE (-1) /* dim exceeds TB_RMSNORM_NOALLOC_MAX_DIM */
#define TB_NOALLOC_ERR_SHAPE (-2)     /* rows < 1, dim not a multiple of the vector width, or unknown dtype */
#define TB_NOALLOC_ERR_SYMBOL (-3)    /* the scratch array's device address could not be obtained */

#ifdef __cplusplus
extern "C" {
#endif

int tb_rmsnorm_bwd_noalloc(const void* g, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                           int rows, int dim, int dtype, cudaStream_t stream);

const char* tb_rmsnorm_bwd_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
