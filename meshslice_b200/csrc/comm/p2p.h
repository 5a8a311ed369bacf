// Stand-alone peer-to-peer collectives over NVLink (all-gather / send-recv by pulling,
// reduce-scatter by pull-and-sum) and the cross-GPU barrier they share with the fused GEMM.
// They are the B200 counterparts of the collectives timed by BenchCollectives2D.py:16-26 and
// feed the cost model's fabric constants.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../gemm/sm100_gemm.h"  // CopyJob, kMaxPeers

namespace msb {

struct BarrierArgs {
  int n_ranks;   // 0: no barrier
  int my_rank;
  uint32_t* entry_flags[kMaxPeers];
  uint32_t* exit_flags[kMaxPeers];
  uint32_t epoch;
  uint32_t* go_flag;       // local
  uint32_t* done_counter;  // local, monotonic
  uint32_t done_target;    // done_counter value once every CTA of this launch has finished
  uint32_t* status;        // [4]
  uint64_t timeout_ns;
};

// Entry barrier, then every CTA copies its share of `jobs` with 16-byte loads from peer memory
// and stores to local memory, then exit barrier (nobody leaves while a peer still reads it).
cudaError_t p2p_copy(const CopyJob* jobs, int n_jobs, const BarrierArgs& bar, int grid,
                     cudaStream_t stream);

// out[r, c] = sum over s of src[s][r, c]  (bf16 in, fp32 sum, bf16 out); src[s] may be peer memory.
struct ReduceArgs {
  const void* src[kMaxPeers];
  int n_src;
  int64_t src_pitch;  // elements
  void* out;
  int64_t out_pitch;  // elements
  int rows, cols;     // cols % 8 == 0
};
cudaError_t p2p_reduce(const ReduceArgs& r, const BarrierArgs& bar, int grid, cudaStream_t stream);

// Only the barrier (one CTA).
cudaError_t p2p_barrier(const BarrierArgs& bar, cudaStream_t stream);

// Test helper for the bounded wait: waits on `flag >= target` for at most timeout_ns, writes
// status[0] = 1 on expiry.  Never spins forever.
cudaError_t bounded_wait_probe(const uint32_t* flag, uint32_t target, uint64_t timeout_ns,
                               uint32_t* status, cudaStream_t stream);

}  // namespace msb
