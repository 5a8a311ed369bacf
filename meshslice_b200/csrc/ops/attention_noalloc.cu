// Attention backward with library-owned scratch (see attention_noalloc.h for who needs it).
#include "attention_noalloc.h"

#include <mutex>

#include "attention.h"

namespace {

constexpr int kHeadDim = 128;
constexpr size_t kAccFloats = (size_t)MSB_NOALLOC_MAX_ROWS * kHeadDim;  // first scratch array of attention_bwd
constexpr size_t kDeltaFloats = MSB_NOALLOC_MAX_ROWS;                   // rowsum(dO * O)
constexpr size_t kStatusFloats = 64;                                    // 4 status words + padding

// One array per device that loads this library.  In host code this name is only a handle for
// cudaGetSymbolAddress; kernels must be given the address that call returns.
static __device__ __align__(256) float g_scratch[kAccFloats + kDeltaFloats + kStatusFloats];

struct PerDevice {
  float* base = nullptr;
};
PerDevice g_dev[64];
std::mutex g_setup_lock;   // first calls from several host threads

}  // namespace

extern "C" cudaError_t msb_attention_bwd_noalloc(const void* qkv, const void* out, const void* dout,
                                                 const float* lse, void* dqkv, int batch, int seq,
                                                 int heads, int causal, float scale,
                                                 cudaStream_t stream, uint32_t* kernel_status) {
  if (batch <= 0 || seq <= 0 || heads <= 0 || seq % 128 != 0) return cudaErrorInvalidValue;
  const long long rows = (long long)batch * seq * heads;
  if (rows > MSB_NOALLOC_MAX_ROWS) return cudaErrorInvalidValue;  // beyond the fixed scratch
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::unique_lock<std::mutex> lock(g_setup_lock);
  if (g_dev[dev].base == nullptr) {
    // set-up, once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scratch);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(p + kAccFloats + kDeltaFloats, 0, kStatusFloats * sizeof(float), stream);
    if (e != cudaSuccess) return e;
    g_dev[dev].base = p;
  }
  lock.unlock();
  float* acc = g_dev[dev].base;
  float* delta = acc + kAccFloats;
  uint32_t* status = reinterpret_cast<uint32_t*>(delta + kDeltaFloats);
  if (kernel_status != nullptr) {
    // status of earlier calls (sticky: never cleared); an async copy into the caller's pinned
    // memory, no allocation
    e = cudaMemcpyAsync(kernel_status, status, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return e;
  }
  // attention_bwd overwrites both scratch arrays (log2-domain lse and the scaled row sums) before it reads them
  return msb::attention_bwd(qkv, out, dout, lse, dqkv, acc, delta, batch, seq, heads, causal, scale,
                            status, stream);
}
