// Two-CTA variant of the local tcgen05 GEMM (no fused collectives): a cluster of two CTAs on
// neighbouring SMs computes one 256 x 256 tile with tcgen05.mma.cta_group::2.
//
// Each CTA loads 128 rows of A and 128 of the 256 B columns per k-block (32 KiB instead of 48 KiB
// per stage, so seven stages fit) and owns the 128 accumulator rows that land in its own TMEM.  Only
// the leader CTA (even rank) issues MMAs; it reads both CTAs' shared memory.  Synchronisation:
//   full[stage]    lives in the leader; both CTAs' TMA loads complete on it (the .cta_group::2
//                  load form with the leader barrier's cluster address); two arrivals: the leader's
//                  A producer and B producer each announce their operand's bytes
//   empty[stage]   one per CTA; the leader commits to its own and to the peer's (mapa address)
//   tfull[acc]     one per CTA, committed by the leader to both
//   tempty[acc]    lives in the leader, 256 arrivals: 128 local, 128 from the peer's epilogue
// No load uses cluster multicast.  Every wait is bounded as in the one-CTA kernel.
#include <cuda_bf16.h>

#include "../common/ptx.cuh"
#include "sm100_gemm.h"

namespace msb {

namespace {

constexpr uint32_t kAStage2 = kBM * kBK * 2;        // 16 KiB: this CTA's 128 rows of A
constexpr uint32_t kBStage2 = (kBN / 2) * kBK * 2;  // 16 KiB: this CTA's 128 columns of B
constexpr uint32_t smem_alloc2(int stages) { return stages * (kAStage2 + kBStage2) + 256 + 1024; }
constexpr int kThreads2 = 224;   // warps: A producer, MMA, 4x epilogue, B producer

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t leader_bar,
                                                 int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t leader_bar,
                                                 int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(leader_bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr)
               : "memory");
}

__device__ __forceinline__ void report2(const GemmArgs& a, uint32_t code, uint32_t d0, uint32_t d1) {
  if (atomicCAS(a.status, 0u, code) == 0u) {
    a.status[1] = blockIdx.x;
    a.status[2] = d0;
    a.status[3] = d1;
  }
}

__device__ __forceinline__ float gelu_tanh2(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}
__device__ __forceinline__ uint32_t pk2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float blo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bhi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

__device__ __forceinline__ void store32(void* base, int64_t ld, bool fp32, bool accumulate, int64_t row,
                                        int col0, int nvalid, float (&v)[32]) {
  if (fp32) {
    float* p = reinterpret_cast<float*>(base) + row * ld + col0;
    if (nvalid == 32) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        if (accumulate) {
          const float4 c = *reinterpret_cast<const float4*>(p + i);
          o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
        }
        *reinterpret_cast<float4*>(p + i) = o;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < nvalid) p[i] = accumulate ? p[i] + v[i] : v[i];
    }
  } else {
    __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(base) + row * ld + col0;
    if (nvalid == 32) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 o;
        if (accumulate) {
          const uint4 c = *reinterpret_cast<const uint4*>(p + i);
          o.x = pk2(v[i] + blo(c.x), v[i + 1] + bhi(c.x));
          o.y = pk2(v[i + 2] + blo(c.y), v[i + 3] + bhi(c.y));
          o.z = pk2(v[i + 4] + blo(c.z), v[i + 5] + bhi(c.z));
          o.w = pk2(v[i + 6] + blo(c.w), v[i + 7] + bhi(c.w));
        } else {
          o.x = pk2(v[i], v[i + 1]);
          o.y = pk2(v[i + 2], v[i + 3]);
          o.z = pk2(v[i + 4], v[i + 5]);
          o.w = pk2(v[i + 6], v[i + 7]);
        }
        *reinterpret_cast<uint4*>(p + i) = o;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (i >= nvalid) continue;
        float x = v[i];
        if (accumulate) x += __bfloat162float(p[i]);
        p[i] = __float2bfloat16_rn(x);
      }
    }
  }
}

// cluster tile t -> (256-row block, 256-column block), grouped along M for L2 reuse
__device__ __forceinline__ void tile2(int t, int tiles_m2, int tiles_n, int group, int& m2, int& nb) {
  const int span = group * tiles_n;
  const int g = t / span;
  const int r = t - g * span;
  const int g0 = g * group;
  const int geff = min(group, tiles_m2 - g0);
  nb = r / geff;
  m2 = g0 + (r - nb * geff);
}

}  // namespace

template <int kStages2>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
sm100_gemm2_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                   const __grid_constant__ GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr uint32_t kSmemB2 = kStages2 * kAStage2;
  constexpr uint32_t kSmemBar2 = kSmemB2 + kStages2 * kBStage2;
  uint8_t* sA = smem;
  uint8_t* sB = smem + kSmemB2;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemBar2);
  uint64_t* full_bar = bars;                    // [kStages2], used in the leader
  uint64_t* empty_bar = bars + kStages2;        // [kStages2], one set per CTA
  uint64_t* tfull_bar = bars + 2 * kStages2;    // [2], one set per CTA
  uint64_t* tempty_bar = tfull_bar + 2;         // [2], used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0: leader
  const uint64_t tmo = a.timeout_ns;
  const int tiles_m2 = (a.M + 2 * kBM - 1) / (2 * kBM);
  const int tiles_n = (a.N + kBN - 1) / kBN;
  const int num_tiles = tiles_m2 * tiles_n;
  const int kblocks = (a.K + kBK - 1) / kBK;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int group = a.group > 0 ? a.group : 8;

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    for (int i = 0; i < kStages2; ++i) {
      mbar_init(full_bar + i, 2);    // the leader's two producers announce their operand's bytes
      mbar_init(empty_bar + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull_bar + i, 1);
      mbar_init(tempty_bar + i, 256);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before_sync();
  cluster_sync_all();      // barriers of both CTAs are initialised before any remote arrival
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 || warp == 6) {
    // ===================== TMA producers (both CTAs): warp 0 loads A, warp 6 loads B ==========
    // One thread issuing every load of a stage is what bounded the tensor pipe with MN-major
    // operands (two boxes per operand): the operands have a producer each, and an MN-major
    // operand is one 3-D box when its extent allows it.
    if (lane == 0) {
      const bool is_a = warp == 0;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += n_clusters) {
        int m2, nb;
        tile2(t, tiles_m2, tiles_n, group, m2, nb);
        const int row_a = (2 * m2 + (int)rank) * kBM;           // this CTA's 128 rows of A
        const int col_b = nb * kBN + (int)rank * (kBN / 2);     // this CTA's 128 columns of B
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar + stage, phase ^ 1, 5 * tmo)) {
            report2(a, kTimeoutEmpty, t, kb);
            ok = false;
            break;
          }
          const uint32_t fb = mapa_u32(smem_u32(full_bar + stage), 0);   // the leader's barrier
          if (is_a) {
            if (rank == 0) mbar_expect_tx(full_bar + stage, 2 * kAStage2);
            uint8_t* da = sA + stage * kAStage2;
            if (!a.a_mn_major) {
              tma_load_2d_pair(da, &tma_a, fb, kb * kBK, row_a);
            } else if (a.a_map3d) {
              tma_load_3d_pair(da, &tma_a, fb, 0, kb * kBK, row_a >> 6);
            } else {
#pragma unroll
              for (int j = 0; j < kBM / 64; ++j)
                tma_load_2d_pair(da + j * (kBK * 128), &tma_a, fb, row_a + j * 64, kb * kBK);
            }
          } else {
            if (rank == 0) mbar_expect_tx(full_bar + stage, 2 * kBStage2);
            uint8_t* db = sB + stage * kBStage2;
            if (!a.b_mn_major) {
              tma_load_2d_pair(db, &tma_b, fb, kb * kBK, col_b);
            } else if (a.b_map3d) {
              tma_load_3d_pair(db, &tma_b, fb, 0, kb * kBK, col_b >> 6);
            } else {
#pragma unroll
              for (int j = 0; j < kBN / 128; ++j)
                tma_load_2d_pair(db + j * (kBK * 128), &tma_b, fb, col_b + j * 64, kb * kBK);
            }
          }
          if (++stage == kStages2) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer (leader only) =====================
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc_bf16(2 * kBM, kBN, a.a_mn_major, a.b_mn_major);
      const uint32_t a_lbo = a.a_mn_major ? kBK * 128 : 16;
      const uint32_t b_lbo = a.b_mn_major ? kBK * 128 : 16;
      const uint32_t a_kstep = a.a_mn_major ? 16 * 128 : 32;
      const uint32_t b_kstep = a.b_mn_major ? 16 * 128 : 32;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = cluster_id; t < num_tiles && ok; t += n_clusters, ++it) {
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar + acc, acc_phase ^ 1, 6 * tmo)) {
          report2(a, kTimeoutTmemEmpty, t, acc);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * kBN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar + stage, phase, 4 * tmo)) {
            report2(a, kTimeoutFull, t, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(sA + stage * kAStage2);
          const uint32_t sb = smem_u32(sB + stage * kBStage2);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = make_smem_desc(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t db = make_smem_desc(sb + k * b_kstep, b_lbo, 1024);
            umma_f16_pair(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          const uint32_t eb = smem_u32(empty_bar + stage);
          umma_commit_pair(eb);                 // this CTA's stage is free
          umma_commit_pair(mapa_u32(eb, 1));    // and the peer's
          if (++stage == kStages2) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          const uint32_t tb = smem_u32(tfull_bar + acc);
          umma_commit_pair(tb);
          umma_commit_pair(mapa_u32(tb, 1));
        }
      }
    }
  } else {
    // ===================== epilogue (both CTAs, own 128 rows) =====================
    const int q = warp & 3;
    const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(a.bias);
    bool ok = true;
    int it = 0;
    for (int t = cluster_id; t < num_tiles && ok; t += n_clusters, ++it) {
      int m2, nb;
      tile2(t, tiles_m2, tiles_n, group, m2, nb);
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
      int okw = 1;
      if (lane == 0) okw = mbar_wait(tfull_bar + acc, acc_phase, 7 * tmo) ? 1 : 0;
      okw = __shfl_sync(0xffffffffu, okw, 0);
      if (!okw) {
        if (lane == 0) report2(a, kTimeoutTmemFull, t, acc);
        ok = false;
        break;
      }
      mbar_wait(tfull_bar + acc, acc_phase, tmo);
      tc_fence_after_sync();
      const int64_t row = (int64_t)(2 * m2 + (int)rank) * kBM + q * 32 + lane;
      const bool row_ok = row < a.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kBN;
      const uint32_t te_leader = mapa_u32(smem_u32(tempty_bar + acc), 0);
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (c == kBN / 32 - 1) {
          tc_fence_before_sync();
          mbar_arrive_cluster(te_leader);     // accumulator drained: tell the leader's MMA warp
        }
        const int col0 = nb * kBN + c * 32;
        const int nvalid = min(32, a.N - col0);
        if (row_ok && nvalid > 0) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < nvalid) v[i] += __bfloat162float(bias[col0 + i]);
          }
          if (a.act == 1) {
            if (a.C_pre != nullptr) store32(a.C_pre, a.ldc, false, false, row, col0, nvalid, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = gelu_tanh2(v[i]);
          }
          store32(a.C, a.ldc, a.c_fp32 != 0, a.accumulate != 0, row, col0, nvalid, v);
        }
      }
    }
  }

  // both CTAs are done with shared memory, barriers and TMEM of the pair
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}

template <int kSt>
static cudaError_t launch2(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const GemmArgs& args, int grid,
                           cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  constexpr int smem = (int)smem_alloc2(kSt);
  if (dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(sm100_gemm2_kernel<kSt>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  // the cluster shape (2,1,1) is part of the kernel's definition
  sm100_gemm2_kernel<kSt><<<grid, kThreads2, smem, stream>>>(tma_a, tma_b, args);
  return cudaGetLastError();
}

cudaError_t launch_sm100_gemm2(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const GemmArgs& args,
                               int grid, cudaStream_t stream) {
  grid &= ~1;
  if (grid < 2) grid = 2;
  if (args.stages == 6) return launch2<6>(tma_a, tma_b, args, grid, stream);
  return launch2<7>(tma_a, tma_b, args, grid, stream);
}

}  // namespace msb
