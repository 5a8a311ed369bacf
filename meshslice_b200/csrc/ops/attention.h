// Flash-style attention for head_dim 128 on tcgen05 tensor cores (score matrix never in HBM).
// Layout of the reference (ShardedLayers.py:152-153): qkv [batch*seq, heads*3*128] with the
// columns of one head ordered [q | k | v]; out / dout [batch*seq, heads*128].
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace msb {

// out = softmax(Q K^T * scale [+ causal mask]) V;  lse[b, h, s] = log sum exp of the scaled scores.
// seq must be a multiple of 128.  status: 4 words, first error wins.
cudaError_t attention_fwd(const void* qkv, void* out, float* lse, int batch, int seq, int heads,
                          int causal, float scale, uint32_t* status, cudaStream_t stream);

// dqkv (same layout as qkv) from dout.  `dq_acc` and `delta` are fp32 scratch of at least
// batch * heads * seq elements each (they receive lse * log2(e) and rowsum(dO * O) * scale); both
// are overwritten.  The gradients are accumulated in tensor memory by the CTA that owns them, so the
// result is bit-identical from run to run.
cudaError_t attention_bwd(const void* qkv, const void* out, const void* dout, const float* lse,
                          void* dqkv, float* dq_acc, float* delta, int batch, int seq, int heads,
                          int causal, float scale, uint32_t* status, cudaStream_t stream);

}  // namespace msb
