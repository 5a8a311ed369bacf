// Peer-to-peer collectives over NVLink with bounded cross-GPU barriers.  See p2p.h.
#include "p2p.h"

#include <cuda_bf16.h>

#include "../common/ptx.cuh"

namespace msb {

namespace {

constexpr uint32_t kErrEntry = 7, kErrExit = 8, kErrGo = 10;

__device__ __forceinline__ void report(uint32_t* status, uint32_t code, uint32_t d0, uint32_t d1) {
  if (atomicCAS(status, 0u, code) == 0u) {
    status[1] = blockIdx.x;
    status[2] = d0;
    status[3] = d1;
  }
}

// All threads of all CTAs call this.  Returns false (uniformly per CTA) on timeout.
__device__ bool barrier_enter(const BarrierArgs& b) {
  if (b.n_ranks <= 0) return true;
  int ok = 1;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    if (blockIdx.x == 0) {
      if (lane < b.n_ranks && lane != b.my_rank) {
        st_release_sys(b.entry_flags[lane] + b.my_rank, b.epoch);
        if (!wait_flag_geq_sys(b.entry_flags[b.my_rank] + lane, b.epoch, b.timeout_ns)) {
          report(b.status, kErrEntry, lane, b.epoch);
          ok = 0;
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (lane == 0 && ok) st_release_gpu(b.go_flag, b.epoch);
    } else if (lane == 0) {
      if (!wait_flag_geq_gpu(b.go_flag, b.epoch, 2 * b.timeout_ns)) {
        report(b.status, kErrGo, 0, b.epoch);
        ok = 0;
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}

// All threads of all CTAs call this after their last access to peer memory.
__device__ void barrier_exit(const BarrierArgs& b, bool ok_in) {
  if (b.n_ranks <= 0) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    red_add_release_gpu(b.done_counter, 1u);
  }
  if (blockIdx.x == 0 && threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int ok = ok_in ? 1 : 0;
    if (lane == 0 && ok) {
      if (!wait_flag_geq_gpu(b.done_counter, b.done_target, 4 * b.timeout_ns)) {
        report(b.status, kErrExit, 0xffffffffu, b.epoch);
        ok = 0;
      }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok && lane < b.n_ranks && lane != b.my_rank) {
      st_release_sys(b.exit_flags[lane] + b.my_rank, b.epoch);
      if (!wait_flag_geq_sys(b.exit_flags[b.my_rank] + lane, b.epoch, 4 * b.timeout_ns))
        report(b.status, kErrExit, lane, b.epoch);
    }
  }
}

__global__ void __launch_bounds__(512)
p2p_copy_kernel(const CopyJob* __restrict__ jobs, int n_jobs, const __grid_constant__ BarrierArgs bar) {
  const bool ok = barrier_enter(bar);
  if (ok) {
    for (int j = 0; j < n_jobs; ++j) {
      const CopyJob job = jobs[j];
      const uint32_t vec_per_row = job.row_bytes >> 4;
      const uint64_t total = (uint64_t)job.rows * vec_per_row;
      const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
      uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
      // four independent 16-byte loads in flight per thread
      for (; i + 3 * stride < total; i += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint64_t k = i + u * stride;
          const uint64_t r = k / vec_per_row, c = k - r * vec_per_row;
          v[u] = *reinterpret_cast<const uint4*>(job.src + r * job.src_pitch + (c << 4));
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint64_t k = i + u * stride;
          const uint64_t r = k / vec_per_row, c = k - r * vec_per_row;
          *reinterpret_cast<uint4*>(job.dst + r * job.dst_pitch + (c << 4)) = v[u];
        }
      }
      for (; i < total; i += stride) {
        const uint64_t r = i / vec_per_row, c = i - r * vec_per_row;
        *reinterpret_cast<uint4*>(job.dst + r * job.dst_pitch + (c << 4)) =
            *reinterpret_cast<const uint4*>(job.src + r * job.src_pitch + (c << 4));
      }
    }
  }
  barrier_exit(bar, ok);
}

__device__ __forceinline__ float lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pk(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(512)
p2p_reduce_kernel(const __grid_constant__ ReduceArgs r, const __grid_constant__ BarrierArgs bar) {
  const bool ok = barrier_enter(bar);
  if (ok) {
    const int vec_per_row = r.cols >> 3;
    const int64_t total = (int64_t)r.rows * vec_per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
      const int64_t row = i / vec_per_row, c = (i - row * vec_per_row) * 8;
      uint4 v[kMaxPeers];
#pragma unroll
      for (int s = 0; s < kMaxPeers; ++s)
        if (s < r.n_src)
          v[s] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(r.src[s]) +
                                                 row * r.src_pitch + c);
      float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int s = 0; s < kMaxPeers; ++s)
        if (s < r.n_src) {
          a[0] += lo(v[s].x); a[1] += hi(v[s].x); a[2] += lo(v[s].y); a[3] += hi(v[s].y);
          a[4] += lo(v[s].z); a[5] += hi(v[s].z); a[6] += lo(v[s].w); a[7] += hi(v[s].w);
        }
      uint4 o;
      o.x = pk(a[0], a[1]); o.y = pk(a[2], a[3]); o.z = pk(a[4], a[5]); o.w = pk(a[6], a[7]);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(r.out) + row * r.out_pitch + c) = o;
    }
  }
  barrier_exit(bar, ok);
}

__global__ void p2p_barrier_kernel(const __grid_constant__ BarrierArgs bar) {
  const bool ok = barrier_enter(bar);
  barrier_exit(bar, ok);
}

__global__ void bounded_wait_probe_kernel(const uint32_t* flag, uint32_t target, uint64_t timeout_ns,
                                          uint32_t* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    if (!wait_flag_geq_sys(flag, target, timeout_ns)) report(status, 1u, target, 0u);
  }
}

}  // namespace

cudaError_t p2p_copy(const CopyJob* jobs, int n_jobs, const BarrierArgs& bar, int grid,
                     cudaStream_t stream) {
  p2p_copy_kernel<<<grid, 512, 0, stream>>>(jobs, n_jobs, bar);
  return cudaGetLastError();
}
cudaError_t p2p_reduce(const ReduceArgs& r, const BarrierArgs& bar, int grid, cudaStream_t stream) {
  if (r.cols % 8 != 0 || r.n_src > kMaxPeers) return cudaErrorInvalidValue;
  p2p_reduce_kernel<<<grid, 512, 0, stream>>>(r, bar);
  return cudaGetLastError();
}
cudaError_t p2p_barrier(const BarrierArgs& bar, cudaStream_t stream) {
  p2p_barrier_kernel<<<1, 32, 0, stream>>>(bar);
  return cudaGetLastError();
}
cudaError_t bounded_wait_probe(const uint32_t* flag, uint32_t target, uint64_t timeout_ns,
                               uint32_t* status, cudaStream_t stream) {
  bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(flag, target, timeout_ns, status);
  return cudaGetLastError();
}

}  // namespace msb
