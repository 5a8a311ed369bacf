// Flash-style attention forward / backward for head_dim 128 on tcgen05 (sm_100a).
//
// Forward, one CTA per (sequence, head, 128 query rows), 192 threads:
//   warp 0     TMA producer: Q once, then K_j / V_j tiles into a two-stage ring
//   warp 1     MMA issuer:   S_j = Q K_j^T into one of two TMEM score buffers, O += P_j V_j
//   warps 2-5  softmax: one thread per query row (TMEM lane); online softmax in the log2 domain
//              with lazy rescaling of O (only when the running maximum grows by more than 2^8),
//              P_j written to shared memory as bf16 in the swizzled operand layout
// Backward, one CTA per (sequence, head, 128 key rows), loop over query blocks:
//   S = Q K^T, dP = dO V^T  ->  P = exp2(S - lse), dS = P (dP - delta) scale  ->
//   dV += P^T dO, dK += dS^T Q (TMEM accumulators), dQ = dS K (added to an fp32 buffer with
//   vector reductions).  All five products read the same shared-memory tiles; only the
//   descriptors (K-major or MN-major view) differ.
// All waits are bounded; a timeout records a code in `status` and the CTA leaves.
#include "attention.h"

#include <cuda_bf16.h>

#include <cstdlib>

#include "../common/ptx.cuh"
#include "../gemm/sm100_gemm.h"  // make_tensor_map_2d

namespace msb {

namespace {

constexpr int kD = 128;         // head dim
constexpr int kBlk = 128;       // query / key rows per tile
constexpr int kTile = kBlk * kD * 2;  // 32 KiB: one [128 x 128] bf16 tile = two swizzle halves
constexpr int kHalf = kTile / 2;
// Element-wise warps (softmax in the forward pass, P / dS and the dQ drain in the backward pass)
// are a template parameter of the kernels.  Four warps give one thread per tile row; eight give
// two threads per row, each owning 64 of the 128 columns: the exponentials and the TMEM traffic
// of a block, which sit in series with the MMAs, take half as long.  A warp may touch the TMEM
// lanes 32 * (warp % 4) ... + 31, so warps 2-5 and 6-9 both cover all four lane quarters.
constexpr int attn_threads(int ew_warps) { return 64 + 32 * ew_warps; }
constexpr uint32_t kErrAttn = 20;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct AttnArgs {
  void* out;          // fwd: out;  bwd: dqkv
  float* lse;
  float* dq_acc;      // bwd
  const float* delta; // bwd
  int batch, seq, heads, causal;
  float scale;
  uint32_t* status;
  uint64_t timeout_ns;
};

__device__ __forceinline__ void report(uint32_t* status, uint32_t code, uint32_t d0, uint32_t d1) {
  if (atomicCAS(status, 0u, code) == 0u) {
    status[1] = blockIdx.x + (blockIdx.y << 12) + (blockIdx.z << 22);
    status[2] = d0;
    status[3] = d1;
  }
}

// Bounded wait that the whole warp follows: lane 0 polls, the verdict is broadcast.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, uint64_t tmo) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, tmo) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (ok) mbar_wait(bar, parity, tmo);  // already complete: orders this lane's later reads
  return ok != 0;
}

// 2^x on the special-function unit in one instruction (relative error 2^-22, denormal results
// flushed to zero: probabilities below 2^-126 are zero anyway).  exp2f() wraps the same
// instruction in range scaling that costs several more issue slots per element.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Writes 32 consecutive columns [c0, c0+32) of row `row` of a [128 x 128] bf16 tile stored as
// two 128-byte-swizzled halves of 64 columns (the layout TMA produces and tcgen05 consumes).
__device__ __forceinline__ void store_tile_row32(uint8_t* tile, int row, int c0, const float (&v)[32]) {
  uint8_t* half = tile + (c0 >> 6) * kHalf + row * 128;
  const int chunk0 = (c0 & 63) >> 3;  // 16-byte chunk index inside the 128-byte row
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 u;
    u.x = pack_bf16(v[q * 8 + 0], v[q * 8 + 1]);
    u.y = pack_bf16(v[q * 8 + 2], v[q * 8 + 3]);
    u.z = pack_bf16(v[q * 8 + 4], v[q * 8 + 5]);
    u.w = pack_bf16(v[q * 8 + 6], v[q * 8 + 7]);
    *reinterpret_cast<uint4*>(half + (((chunk0 + q) ^ (row & 7)) << 4)) = u;
  }
}

// K-major view of a tile: rows = M or N index, contraction along the 128 columns.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int kstep) {
  return make_smem_desc(tile + (kstep >> 2) * kHalf + (kstep & 3) * 32, 16, 1024);
}
// MN-major view: rows = contraction index (16 per step), the 128 columns are the M or N index.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int kstep) {
  return make_smem_desc(tile + kstep * 2048, kHalf, 1024);
}

__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int col,
                                          int row) {
  tma_load_2d(dst, map, bar, col, row);
  tma_load_2d(dst + kHalf, map, bar, col + 64, row);
}

// ==========================================================================================
// forward
// ==========================================================================================
template <int kEwWarps>
__global__ void __launch_bounds__(attn_threads(kEwWarps), 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ AttnArgs a) {
  static_assert(kEwWarps == 4 || kEwWarps == 8, "four or eight element-wise warps");
  constexpr int kHalves = kEwWarps / 4;
  constexpr int kColsPer = kBlk / kHalves;   // columns per thread
  constexpr int kChunks = kColsPer / 32;     // 32-column TMEM loads per thread and block
  constexpr int kEwThreads = 32 * kEwWarps;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTile;            // 2 stages
  uint8_t* sV = smem + 3 * kTile;        // 2 stages
  uint8_t* sP = smem + 5 * kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTile);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;    // [2]
  uint64_t* p_ready = bars + 7;
  uint64_t* pv_done = bars + 8;
  uint64_t* xchg = bars + 9;      // the two threads of a row exchange their partial maximum / sum
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  float* sX = reinterpret_cast<float*>(smem + 6 * kTile + 256);   // [2 phases][2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = a.seq / kBlk;
  const int i_blk = a.causal ? (nblk - 1 - (int)blockIdx.x) : (int)blockIdx.x;  // heavy tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int n_kv = a.causal ? i_blk + 1 : nblk;
  const int row0 = b * a.seq + i_blk * kBlk;
  const int colq = h * 3 * kD;
  const uint64_t tmo = a.timeout_ns;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm_qkv);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(kv_full + i, 1);
      mbar_init(kv_empty + i, 1);
      mbar_init(s_full + i, 1);
    }
    mbar_init(p_ready, kEwThreads);
    mbar_init(pv_done, 1);
    mbar_init(xchg, kEwThreads);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_o = tmem + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, kTile);
      load_tile(sQ, &tm_qkv, q_full, colq, row0);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait(kv_empty + st, ((j >> 1) & 1) ^ 1, 4 * tmo)) {
          report(a.status, kErrAttn + 1, j, 0);
          break;
        }
        mbar_expect_tx(kv_full + st, 2 * kTile);
        const int krow = b * a.seq + j * kBlk;
        load_tile(sK + st * kTile, &tm_qkv, kv_full + st, colq + kD, krow);
        load_tile(sV + st * kTile, &tm_qkv, kv_full + st, colq + 2 * kD, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, 128, 0, 1);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, 2 * tmo) && mbar_wait(kv_full, 0, 2 * tmo);
      if (!ok) report(a.status, kErrAttn + 2, 0, 0);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(sK);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16(tmem, desc_kmajor(q_addr, k), desc_kmajor(k_addr, k), idesc_s, k != 0);
        umma_commit(s_full);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const int st = (j + 1) & 1;
          if (!mbar_wait(kv_full + st, ((j + 1) >> 1) & 1, 2 * tmo)) {
            report(a.status, kErrAttn + 3, j, 0);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t k_addr = smem_u32(sK + st * kTile);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_f16(tmem + st * 128, desc_kmajor(q_addr, k), desc_kmajor(k_addr, k), idesc_s, k != 0);
          umma_commit(s_full + st);
        }
        if (!mbar_wait(p_ready, j & 1, 4 * tmo)) {
          report(a.status, kErrAttn + 4, j, 0);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(sV + (j & 1) * kTile);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16(tmem_o, desc_kmajor(p_addr, k), desc_mnmajor(v_addr, k), idesc_pv, (j | k) != 0);
        umma_commit(pv_done);
        umma_commit(kv_empty + (j & 1));
      }
    }
  } else {
    // ---------------- softmax / epilogue: kHalves threads per query row ----------------
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;         // which kColsPer columns of the row this thread owns
    const int col0 = half * kColsPer;
    const int row = q4 * 32 + lane;           // row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    const float sl2 = a.scale * kLog2e;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    int xphase = 0;
    // both threads of a row leave this with the combined value (maximum or sum)
    auto exchange = [&](float v, bool is_max, bool& good) -> float {
      if (kHalves == 1) return v;
      sX[(xphase * 2 + half) * kBlk + row] = v;
      mbar_arrive(xchg);
      if (!warp_wait(xchg, xphase, 6 * tmo)) {
        good = false;
        return v;
      }
      const float o = sX[(xphase * 2 + (half ^ 1)) * kBlk + row];
      xphase ^= 1;
      return is_max ? fmaxf(v, o) : v + o;
    };
    for (int j = 0; j < n_kv; ++j) {
      const int sb = j & 1;
      if (!warp_wait(s_full + sb, (j >> 1) & 1, 6 * tmo)) {
        if (lane == 0) report(a.status, kErrAttn + 5, j, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t ts = tmem + lane_off + sb * 128 + col0;
      const bool diag = a.causal && j == i_blk;
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(ts + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float v = __uint_as_float(r[i]);
          if (!diag || col0 + c * 32 + i <= row) mx = fmaxf(mx, v);
        }
      }
      mx = exchange(mx, true, ok);
      if (!ok) {
        if (lane == 0) report(a.status, kErrAttn + 8, j, 0);
        break;
      }
      const float m_blk = mx * sl2;
      if (j == 0) {
        m_used = m_blk;
      } else {
        // P of the previous block has been consumed and O is up to date after this wait
        if (!warp_wait(pv_done, (j - 1) & 1, 6 * tmo)) {
          if (lane == 0) report(a.status, kErrAttn + 6, j, 0);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const float m_new = fmaxf(m_used, m_blk);
        const bool need = (m_new - m_used) > 8.0f;
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = need ? exp2f(m_used - m_new) : 1.0f;
          if (need) {
            l *= alpha;
            m_used = m_new;
          }
          const uint32_t to = tmem_o + lane_off + col0;
#pragma unroll 1
          for (int c = 0; c < kChunks; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(to + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(to + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      float rowsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(ts + c * 32, r);
        tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = fast_exp2(__uint_as_float(r[i]) * sl2 - m_used);
          if (diag && col0 + c * 32 + i > row) e = 0.f;
          p[i] = e;
          rowsum += e;
        }
        store_tile_row32(sP, row, col0 + c * 32, p);
      }
      l += rowsum;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(p_ready);
    }
    if (ok) {
      l = exchange(l, false, ok);   // the row's denominator: both halves
      if (!ok && lane == 0) report(a.status, kErrAttn + 9, 0, 0);
    }
    if (ok) {
      if (!warp_wait(pv_done, (n_kv - 1) & 1, 6 * tmo)) {
        if (lane == 0) report(a.status, kErrAttn + 7, 0, 0);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.0f / l;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(a.out) +
                            (int64_t)(row0 + row) * (a.heads * kD) + h * kD + col0;
      const uint32_t to = tmem_o + lane_off + col0;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(to + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 u;
          u.x = pack_bf16(__uint_as_float(r[q * 8 + 0]) * inv, __uint_as_float(r[q * 8 + 1]) * inv);
          u.y = pack_bf16(__uint_as_float(r[q * 8 + 2]) * inv, __uint_as_float(r[q * 8 + 3]) * inv);
          u.z = pack_bf16(__uint_as_float(r[q * 8 + 4]) * inv, __uint_as_float(r[q * 8 + 5]) * inv);
          u.w = pack_bf16(__uint_as_float(r[q * 8 + 6]) * inv, __uint_as_float(r[q * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = u;
        }
      }
      if (half == 0) a.lse[((int64_t)b * a.heads + h) * a.seq + i_blk * kBlk + row] = m_used * kLn2 + logf(l);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ==========================================================================================
// backward
// ==========================================================================================
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int batch, int seq, int heads) {
  // one warp per (token, head): delta = sum_d out * dout
  const int64_t w = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t total = (int64_t)batch * seq * heads;
  if (w >= total) return;
  const int64_t t = w / heads;
  const int h = (int)(w - t * heads);
  const uint2 o = *reinterpret_cast<const uint2*>(out + t * heads * kD + h * kD + lane * 4);
  const uint2 d = *reinterpret_cast<const uint2*>(dout + t * heads * kD + h * kD + lane * 4);
  float s = __uint_as_float(o.x << 16) * __uint_as_float(d.x << 16) +
            __uint_as_float(o.x & 0xffff0000u) * __uint_as_float(d.x & 0xffff0000u) +
            __uint_as_float(o.y << 16) * __uint_as_float(d.y << 16) +
            __uint_as_float(o.y & 0xffff0000u) * __uint_as_float(d.y & 0xffff0000u);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) {
    const int64_t bq = t / seq, sq = t - bq * seq;
    delta[(bq * heads + h) * seq + sq] = s;
  }
}

__global__ void attn_dq_store_kernel(const float4* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv,
                                     int64_t tokens, int heads) {
  const int64_t nvec = tokens * heads * (kD / 4);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t th = i / (kD / 4);
    const int v = (int)(i - th * (kD / 4));
    const int64_t t = th / heads;
    const int h = (int)(th - t * heads);
    const float4 f = dq_acc[i];
    uint2 o;
    o.x = pack_bf16(f.x, f.y);
    o.y = pack_bf16(f.z, f.w);
    *reinterpret_cast<uint2*>(dqkv + t * heads * 3 * kD + h * 3 * kD + v * 4) = o;
  }
}

template <int kEwWarps>
__global__ void __launch_bounds__(attn_threads(kEwWarps), 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ AttnArgs a) {
  static_assert(kEwWarps == 4 || kEwWarps == 8, "four or eight element-wise warps");
  constexpr int kColsPer = kBlk / (kEwWarps / 4);
  constexpr int kChunks = kColsPer / 32;
  constexpr int kEwThreads = 32 * kEwWarps;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTile;
  uint8_t* sQ = smem + 2 * kTile;
  uint8_t* sdO = smem + 3 * kTile;
  uint8_t* sP = smem + 4 * kTile;
  uint8_t* sdS = smem + 5 * kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTile);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* pds_ready = bars + 4;
  uint64_t* mma_done = bars + 5;
  uint64_t* dq_drained = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = a.seq / kBlk;
  const int j_blk = blockIdx.x;   // key block; with a causal mask low j means more work: first
  const int h = blockIdx.y, b = blockIdx.z;
  const int i0 = a.causal ? j_blk : 0;
  const int n_it = nblk - i0;
  const int colq = h * 3 * kD;
  const uint64_t tmo = a.timeout_ns;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm_qkv);
    tma_prefetch_desc(&tm_do);
    mbar_init(kv_full, 1);
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, kEwThreads);
    mbar_init(mma_done, 1);
    mbar_init(dq_drained, kEwThreads);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_s = tmem, t_dp = tmem + 128, t_dv = tmem + 256, t_dk = tmem + 384;

  if (warp == 0) {
    if (lane == 0) {
      const int krow = b * a.seq + j_blk * kBlk;
      mbar_expect_tx(kv_full, 2 * kTile);
      load_tile(sK, &tm_qkv, kv_full, colq + kD, krow);
      load_tile(sV, &tm_qkv, kv_full, colq + 2 * kD, krow);
      for (int it = 0; it < n_it; ++it) {
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1, 6 * tmo)) {
          report(a.status, kErrAttn + 11, it, 0);
          break;
        }
        const int qrow = b * a.seq + (i0 + it) * kBlk;
        mbar_expect_tx(qdo_full, 2 * kTile);
        load_tile(sQ, &tm_qkv, qdo_full, colq, qrow);
        load_tile(sdO, &tm_do, qdo_full, h * kD, qrow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_kk = make_idesc_bf16(128, 128, 0, 0);   // both operands K-major
      const uint32_t id_mm = make_idesc_bf16(128, 128, 1, 1);   // both MN-major
      const uint32_t id_km = make_idesc_bf16(128, 128, 0, 1);   // A K-major, B MN-major
      const uint32_t k_a = smem_u32(sK), v_a = smem_u32(sV), q_a = smem_u32(sQ), do_a = smem_u32(sdO),
                     p_a = smem_u32(sP), ds_a = smem_u32(sdS);
      bool ok = mbar_wait(kv_full, 0, 2 * tmo);
      if (!ok) report(a.status, kErrAttn + 12, 0, 0);
      for (int it = 0; it < n_it && ok; ++it) {
        if (!mbar_wait(qdo_full, it & 1, 2 * tmo) || !mbar_wait(dq_drained, (it & 1) ^ 1, 6 * tmo)) {
          report(a.status, kErrAttn + 13, it, 0);
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k)   // S = Q K^T
          umma_f16(t_s, desc_kmajor(q_a, k), desc_kmajor(k_a, k), id_kk, k != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)   // dP = dO V^T
          umma_f16(t_dp, desc_kmajor(do_a, k), desc_kmajor(v_a, k), id_kk, k != 0);
        umma_commit(sdp_full);
        if (!mbar_wait(pds_ready, it & 1, 6 * tmo)) {
          report(a.status, kErrAttn + 14, it, 0);
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k)   // dV += P^T dO   (contraction over the query rows)
          umma_f16(t_dv, desc_mnmajor(p_a, k), desc_mnmajor(do_a, k), id_mm, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)   // dK += dS^T Q
          umma_f16(t_dk, desc_mnmajor(ds_a, k), desc_mnmajor(q_a, k), id_mm, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)   // dQ = dS K      (contraction over the key rows)
          umma_f16(t_s, desc_kmajor(ds_a, k), desc_mnmajor(k_a, k), id_km, k != 0);
        umma_commit(mma_done);
        umma_commit(qdo_empty);
      }
    }
  } else {
    const int q4 = warp & 3;
    const int col0 = ((warp - 2) >> 2) * kColsPer;   // this thread's columns of every 128-wide row
    const int row = q4 * 32 + lane;
    const uint32_t lane_off = (static_cast<uint32_t>(q4 * 32) << 16) + col0;
    const float sl2 = a.scale * kLog2e;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int i_blk = i0 + it;
      const int64_t qtok = (int64_t)b * a.seq + i_blk * kBlk + row;
      const int64_t sidx = ((int64_t)b * a.heads + h) * a.seq + i_blk * kBlk + row;
      const float lse2 = a.lse[sidx] * kLog2e;
      const float dlt = a.delta[sidx];
      if (!warp_wait(sdp_full, it & 1, 8 * tmo)) {
        if (lane == 0) report(a.status, kErrAttn + 15, it, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const bool diag = a.causal && i_blk == j_blk;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(t_s + lane_off + c * 32, rs);
        tmem_ld_32x32(t_dp + lane_off + c * 32, rp);
        tmem_ld_wait();
        float p[32], ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = fast_exp2(__uint_as_float(rs[i]) * sl2 - lse2);
          if (diag && col0 + c * 32 + i > row) e = 0.f;
          p[i] = e;
          ds[i] = e * (__uint_as_float(rp[i]) - dlt) * a.scale;
        }
        store_tile_row32(sP, row, col0 + c * 32, p);
        store_tile_row32(sdS, row, col0 + c * 32, ds);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(pds_ready);
      if (!warp_wait(mma_done, it & 1, 8 * tmo)) {
        if (lane == 0) report(a.status, kErrAttn + 16, it, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      float* dq = a.dq_acc + qtok * (a.heads * kD) + h * kD + col0;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_s + lane_off + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq + c * 32 + q * 4),
                       "f"(__uint_as_float(r[q * 4 + 0])), "f"(__uint_as_float(r[q * 4 + 1])),
                       "f"(__uint_as_float(r[q * 4 + 2])), "f"(__uint_as_float(r[q * 4 + 3]))
                       : "memory");
        }
      }
      tc_fence_before_sync();
      mbar_arrive(dq_drained);
    }
    if (ok) {
      // dV and dK of this key block are complete (mma_done of the last iteration was awaited)
      __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(a.out) +
                            ((int64_t)b * a.seq + j_blk * kBlk + row) * (a.heads * 3 * kD) + colq;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t t = (which == 0 ? t_dk : t_dv) + lane_off;
        __nv_bfloat16* dst = base + (which == 0 ? kD : 2 * kD) + col0;
#pragma unroll 1
        for (int c = 0; c < kChunks; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1]));
            u.y = pack_bf16(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
            u.z = pack_bf16(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]));
            u.w = pack_bf16(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = u;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

constexpr size_t kAttnSmem = 6 * kTile + 256 + 2 * 2 * kBlk * sizeof(float) + 1024;

// Element-wise warps per CTA: 8 unless MSB_ATTN_EW_WARPS=4 is set in the environment.
int ew_warps() {
  static const int v = [] {
    const char* e = std::getenv("MSB_ATTN_EW_WARPS");
    return (e != nullptr && e[0] == '4' && e[1] == '\0') ? 4 : 8;
  }();
  return v;
}

// The shared-memory attribute is per device: set it once on every device that launches.
cudaError_t configure_device() {
  static bool configured[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && configured[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(attn_fwd_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnSmem);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(attn_fwd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnSmem);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(attn_bwd_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnSmem);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(attn_bwd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnSmem);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64) configured[dev] = true;
  return cudaSuccess;
}

}  // namespace

cudaError_t attention_fwd(const void* qkv, void* out, float* lse, int batch, int seq, int heads,
                          int causal, float scale, uint32_t* status, cudaStream_t stream) {
  if (seq % kBlk != 0 || batch <= 0 || heads <= 0) return cudaErrorInvalidValue;
  {
    cudaError_t e = configure_device();
    if (e != cudaSuccess) return e;
  }
  CUtensorMap tm;
  const uint64_t width = (uint64_t)heads * 3 * kD;
  if (make_tensor_map_2d(&tm, qkv, width, (uint64_t)batch * seq, width * 2, 64, kBlk) != 0)
    return cudaErrorInvalidValue;
  AttnArgs a{};
  a.out = out;
  a.lse = lse;
  a.batch = batch; a.seq = seq; a.heads = heads; a.causal = causal;
  a.scale = scale;
  a.status = status;
  a.timeout_ns = 2000000000ull;
  dim3 grid(seq / kBlk, heads, batch);
  if (ew_warps() == 8) attn_fwd_kernel<8><<<grid, attn_threads(8), kAttnSmem, stream>>>(tm, a);
  else attn_fwd_kernel<4><<<grid, attn_threads(4), kAttnSmem, stream>>>(tm, a);
  return cudaGetLastError();
}

cudaError_t attention_bwd(const void* qkv, const void* out, const void* dout, const float* lse,
                          void* dqkv, float* dq_acc, float* delta, int batch, int seq, int heads,
                          int causal, float scale, uint32_t* status, cudaStream_t stream) {
  if (seq % kBlk != 0 || batch <= 0 || heads <= 0) return cudaErrorInvalidValue;
  {
    cudaError_t e0 = configure_device();
    if (e0 != cudaSuccess) return e0;
  }
  const int64_t tokens = (int64_t)batch * seq;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, tokens * heads * kD * sizeof(float), stream);
  if (e != cudaSuccess) return e;
  {
    const int64_t warps = tokens * heads;
    const int threads = 256;
    const int64_t blocks = (warps * 32 + threads - 1) / threads;
    attn_delta_kernel<<<(unsigned)blocks, threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout), delta, batch, seq, heads);
  }
  CUtensorMap tq, td;
  const uint64_t width = (uint64_t)heads * 3 * kD, wdo = (uint64_t)heads * kD;
  if (make_tensor_map_2d(&tq, qkv, width, (uint64_t)tokens, width * 2, 64, kBlk) != 0) return cudaErrorInvalidValue;
  if (make_tensor_map_2d(&td, dout, wdo, (uint64_t)tokens, wdo * 2, 64, kBlk) != 0) return cudaErrorInvalidValue;
  AttnArgs a{};
  a.out = dqkv;
  a.lse = const_cast<float*>(lse);
  a.dq_acc = dq_acc;
  a.delta = delta;
  a.batch = batch; a.seq = seq; a.heads = heads; a.causal = causal;
  a.scale = scale;
  a.status = status;
  a.timeout_ns = 2000000000ull;
  dim3 grid(seq / kBlk, heads, batch);
  if (ew_warps() == 8) attn_bwd_kernel<8><<<grid, attn_threads(8), kAttnSmem, stream>>>(tq, td, a);
  else attn_bwd_kernel<4><<<grid, attn_threads(4), kAttnSmem, stream>>>(tq, td, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  attn_dq_store_kernel<<<148 * 8, 256, 0, stream>>>(reinterpret_cast<const float4*>(dq_acc),
                                                   reinterpret_cast<__nv_bfloat16*>(dqkv), tokens, heads);
  return cudaGetLastError();
}

}  // namespace msb
