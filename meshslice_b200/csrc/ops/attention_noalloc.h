// Attention backward for callers that must not allocate.
//
// This entry point has no counterpart in the reference.  It exists for hosts that embed the
// library where device allocation is off limits at call time: code running under a memory
// budget fixed at start-up, plugins handed only their input and output buffers, and anything
// that must not disturb another allocator's pool.  The regular attention_bwd needs two scratch
// buffers from its caller; here they live in a fixed array inside the library instead.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem accepted: batch * seq * heads <= MSB_NOALLOC_MAX_ROWS (the scratch holds
// 128 fp32 per such row plus one fp32 per row, about 8.1 MiB, resident on every GPU that loads
// the library until the process exits).
#define MSB_NOALLOC_MAX_ROWS 16384

// Same result as msb::attention_bwd: dqkv (layout of qkv) from dout, out and lse.
//   * Nothing is allocated: no cudaMalloc / cudaFree and no allocating library call.
//   * The first call on a device looks up the scratch array's device address
//     (cudaGetSymbolAddress) and sets the kernels' shared-memory attribute; make that first
//     call outside any stream capture.
//   * All calls share one scratch array per device.  Each call clears what it needs, so calls
//     may follow each other on one stream, but two calls that overlap on the GPU (different
//     streams) race on it.
//   * The set-up is serialised by a lock, so first calls from several host threads are safe;
//     the device is the one current in the calling thread.
// Returns cudaErrorInvalidValue when the problem exceeds MSB_NOALLOC_MAX_ROWS or seq is not a
// multiple of 128; otherwise the launch status.
// kernel_status (may be null) must point to PINNED host memory (cudaHostAlloc / cudaHostRegister):
// the bounded-wait status word of the kernels is copied there asynchronously on `stream`, ordered
// before this call's kernels, so after the stream has run it holds what EARLIER calls on this
// device reported (0 = ok).  The word is sticky: the first error code stays until the process
// exits, later calls report it again.  With pageable memory the copy would block the host, and a
// copy to host memory is not allowed while `stream` is being captured: pass null in both cases.
cudaError_t msb_attention_bwd_noalloc(const void* qkv, const void* out, const void* dout,
                                      const float* lse, void* dqkv, int batch, int seq, int heads,
                                      int causal, float scale, cudaStream_t stream,
                                      uint32_t* kernel_status);

#ifdef __cplusplus
}
#endif
