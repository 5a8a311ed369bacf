// Flash-style attention forward / backward for head_dim 128 on tcgen05 (sm_100a): the score matrix
// lives in tensor memory only.
//
// Forward (attn_fwd2_kernel): one CTA per (sequence, head, 128 query rows), two CTAs per SM; S = Q K^T
//   into TMEM, online softmax in the log2 domain with lazy rescaling of O (only when the running
//   maximum grows by more than 2^8), P written back over S as packed bf16 and read by O += P V as
//   the TMEM operand.
// Backward (attn_bwd2_kernel<key-major>, <query-major>): dK / dV are accumulated by the CTA that owns
//   128 keys, dQ by the CTA that owns 128 queries; both recompute S and dP, keep P and dS in TMEM,
//   and never add to global memory: the gradients are bit-identical from run to run.
// All waits are bounded; a timeout records a code in `status` and the CTA leaves.
#include "attention.h"

#include <cuda_bf16.h>

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
// forward: P stays in tensor memory, two CTAs per SM
// ==========================================================================================
// One CTA per (sequence, head, 128 query rows), sized so that TWO CTAs share an SM
// (96 KiB of shared memory, 256 TMEM columns, 192 threads each): while one CTA's softmax runs on the
// SIMT pipes the other's products keep the tensor pipe busy, without any hand-written ping-pong.
//   warp 0     TMA producer: Q once; K_j and V_j into one buffer each (K_{j+1} travels under
//              softmax(j) and P V(j), V_{j+1} under S(j+1) and softmax(j+1))
//   warp 1     MMA issuer: S_j = Q K_j^T into TMEM columns [0,128); O += P_j V_j with P_j read from
//              TMEM (the A operand of tcgen05.mma may live in tensor memory), V_j from shared memory
//   warps 2-5  softmax: one thread per query row; two passes over S in TMEM (row maximum, then
//              exponentials); P_j is written back over S as packed bf16 (64 columns), so it never
//              touches shared memory and needs no proxy fence
// The tensor pipe runs the MMAs of a CTA in issue order, so S_{j+1} may be issued right behind
// P_j V_j although it overwrites P_j, and a completed S_{j+1} implies a completed P_j V_j (O is safe
// to rescale).
constexpr size_t kFwd2Smem = 3 * kTile + 256 + 1024;

__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp writes row (lane base + t).
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__global__ void __launch_bounds__(192, 2)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTile;
  uint8_t* sV = smem + 2 * kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * kTile);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;
  uint64_t* o_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = a.seq / kBlk;
  // Grid = (batch-heads of a group, tiles, groups): blocks are handed to the SMs in block-id order, so a group of
  // up to 32 batch-heads (whose Q / K / V stay in L2 together) runs its longest causal tiles first and the last
  // wave of the launch is the short tiles.
  const int i_blk = a.causal ? (nblk - 1 - (int)blockIdx.y) : (int)blockIdx.y;
  const int bh = blockIdx.z * gridDim.x + blockIdx.x;
  const int h = bh % a.heads, b = bh / a.heads;
  const int n_kv = a.causal ? i_blk + 1 : nblk;
  const int row0 = b * a.seq + i_blk * kBlk;
  const int colq = h * 3 * kD;
  const uint64_t tmo = a.timeout_ns;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm_qkv);
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_o = tmem + 128;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, kTile);
      load_tile(sQ, &tm_qkv, q_full, colq, row0);
      for (int j = 0; j < n_kv; ++j) {
        const int krow = b * a.seq + j * kBlk;
        if (!mbar_wait(k_empty, (j & 1) ^ 1, 4 * tmo)) {
          report(a.status, kErrAttn + 1, j, 0);
          break;
        }
        mbar_expect_tx(k_full, kTile);
        load_tile(sK, &tm_qkv, k_full, colq + kD, krow);
        if (!mbar_wait(v_empty, (j & 1) ^ 1, 4 * tmo)) {
          report(a.status, kErrAttn + 1, j, 1);
          break;
        }
        mbar_expect_tx(v_full, kTile);
        load_tile(sV, &tm_qkv, v_full, colq + 2 * kD, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, 128, 0, 1);
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      // Every product of this CTA reads the same three buffers: all 24 operand descriptors are
      // built once.  One thread issues every MMA, and an MMA of this size occupies the tensor pipe
      // for about 64 cycles: building descriptors in the loop would make the issue the bottleneck.
      uint64_t dq[8], dkk[8], dv[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        dq[k] = desc_kmajor(q_addr, k);
        dkk[k] = desc_kmajor(k_addr, k);
        dv[k] = desc_mnmajor(v_addr, k);
      }
      bool ok = mbar_wait(q_full, 0, 2 * tmo) && mbar_wait(k_full, 0, 2 * tmo);
      if (!ok) report(a.status, kErrAttn + 2, 0, 0);
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tmem, dq[k], dkk[k], idesc_s, k != 0);
        umma_commit(s_full);
        umma_commit(k_empty);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (!mbar_wait(p_ready, j & 1, 6 * tmo) || !mbar_wait(v_full, j & 1, 2 * tmo)) {
          report(a.status, kErrAttn + 4, j, 0);
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k)   // 16 bf16 of a row of P = 8 TMEM columns per step
          umma_f16_ts(tmem_o, tmem + k * 8, dv[k], idesc_pv, (j | k) != 0);
        umma_commit(v_empty);
        if (j + 1 == n_kv) {
          umma_commit(o_done);
        } else {
          if (!mbar_wait(k_full, (j + 1) & 1, 2 * tmo)) {
            report(a.status, kErrAttn + 3, j, 0);
            ok = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16(tmem, dq[k], dkk[k], idesc_s, k != 0);
          umma_commit(s_full);
          umma_commit(k_empty);
        }
      }
    }
  } else {
    // ---------------- softmax / epilogue: one thread per query row ----------------
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;           // row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    const uint32_t ts = tmem + lane_off, to = tmem_o + lane_off;
    const float sl2 = a.scale * kLog2e;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!warp_wait(s_full, j & 1, 6 * tmo)) {
        if (lane == 0) report(a.status, kErrAttn + 5, j, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const bool diag = a.causal && j == i_blk;
      float mx = -INFINITY;
      // the masked forms run for the diagonal block only: the other blocks carry no mask arithmetic
      if (!diag) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(ts + c * 32, r);
          tmem_ld_wait();
          float m0 = __uint_as_float(r[0]), m1 = __uint_as_float(r[1]);
#pragma unroll
          for (int i = 2; i < 32; i += 2) {
            m0 = fmaxf(m0, __uint_as_float(r[i]));
            m1 = fmaxf(m1, __uint_as_float(r[i + 1]));
          }
          mx = fmaxf(mx, fmaxf(m0, m1));
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(ts + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i <= row) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      }
      const float m_blk = mx * sl2;
      if (j == 0) {
        m_used = m_blk;
      } else {
        // S_j is complete, hence P_{j-1} V_{j-1} is too: O may be rescaled in place
        const float m_new = fmaxf(m_used, m_blk);
        const bool need = (m_new - m_used) > 8.0f;
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = need ? exp2f(m_used - m_new) : 1.0f;
          if (need) {
            l *= alpha;
            m_used = m_new;
          }
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(to + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(to + c * 32, r);
          }
        }
      }
      float rowsum = 0.f;
      const float neg_m = -m_used;
      if (!diag) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32], pk[16];
          tmem_ld_32x32(ts + c * 32, r);
          tmem_ld_wait();
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = fast_exp2(fmaf(__uint_as_float(r[i]), sl2, neg_m));
            const float e1 = fast_exp2(fmaf(__uint_as_float(r[i + 1]), sl2, neg_m));
            s0 += e0;
            s1 += e1;
            pk[i >> 1] = pack_bf16(e0, e1);
          }
          rowsum += s0 + s1;
          // P columns [32c, 32c+32) as bf16 = TMEM columns [16c, 16c+16): over S columns already read
          tmem_st_32x16(ts + c * 16, pk);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32], pk[16];
          tmem_ld_32x32(ts + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float e0 = fast_exp2(fmaf(__uint_as_float(r[i]), sl2, neg_m));
            float e1 = fast_exp2(fmaf(__uint_as_float(r[i + 1]), sl2, neg_m));
            if (c * 32 + i > row) e0 = 0.f;
            if (c * 32 + i + 1 > row) e1 = 0.f;
            rowsum += e0 + e1;
            pk[i >> 1] = pack_bf16(e0, e1);
          }
          tmem_st_32x16(ts + c * 16, pk);
        }
      }
      l += rowsum;
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(p_ready);
    }
    if (ok) {
      if (!warp_wait(o_done, 0, 6 * tmo)) {
        if (lane == 0) report(a.status, kErrAttn + 7, 0, 0);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.0f / l;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(a.out) +
                            (int64_t)(row0 + row) * (a.heads * kD) + h * kD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
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
      a.lse[((int64_t)b * a.heads + h) * a.seq + i_blk * kBlk + row] = m_used * kLn2 + logf(l);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem, 256);
}

// ==========================================================================================
// backward
// ==========================================================================================
// delta[b, h, s] = rowsum(dO * O) * scale and lse2[b, h, s] = lse * log2(e): pre-scaled so that the
// element-wise passes of the backward kernels need one fused multiply-add each for the exponent and
// for dP * scale - delta.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int batch, int seq, int heads,
                                  const float* __restrict__ lse, float* __restrict__ lse2, float scale) {
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
    const int64_t idx = (bq * heads + h) * seq + sq;
    delta[idx] = s * scale;
    lse2[idx] = lse[idx] * kLog2e;
  }
}

// ==========================================================================================
// backward: two deterministic kernels, P / dS stay in tensor memory
// ==========================================================================================
// The gradient is split by who accumulates it:
//   attn_bwd2_kernel<true>   one CTA per 128 KEYS walks the query blocks and accumulates dV, dK in TMEM
//   attn_bwd2_kernel<false>  one CTA per 128 QUERIES walks the key blocks and accumulates dQ in TMEM
// Both recompute S and dP (7 products per block pair instead of 5), but nothing is ever added to
// global memory: no fp32 dQ buffer, no memset, no atomics, and the result is bit-identical from run
// to run.  P and dS are written back over S and dP as packed bf16 and feed the gradient products
// as the TMEM (A) operand: they never touch shared memory.
//
// An MMA of M = 128 occupies the tensor pipe for about 92-105 cycles whatever its N up to 128, so
// the products use full 128-wide blocks (eight instructions each) and the kernels are organised
// around keeping that one pipe fed: the element-wise work is split in two phases (P from S; dS from
// dP and P) and the MMA warp issues the next block's S (and dP) between the gradient products of the
// current block, so each phase runs under products that do not depend on it:
//   key-major    S(i) dP(i) | P(i)? dV(i) S(i+1) | dS(i)? dK(i) dP(i+1) | P(i+1)? ...
//   query-major  S(j) dP(j) S(j+1) | dS(j)? dQ(j) dP(j+1) S(j+2) | ...          (two S buffers)
//
//   warp 0      TMA: the two resident 128-row tiles once, then a two-stage ring of 128-row tile pairs
//   warp 1      MMA issuer (all operand descriptors are built once, outside the loops)
//   warps 2-9   element-wise: two threads per TMEM lane, 64 of the 128 columns each
constexpr int kRing = 2;
constexpr size_t kBwd2Smem = 2 * kTile + kRing * 2 * kTile + 256 + 1024;
constexpr int kBwd2Threads = 64 + 32 * 8;

struct Bwd2Args {
  void* dqkv;
  const float* lse2;    // lse * log2(e)          (written by attn_delta_kernel)
  const float* delta;   // rowsum(dO * O) * scale (written by attn_delta_kernel)
  int batch, seq, heads, causal;
  float scale;
  uint32_t* status;
  uint64_t timeout_ns;
};

// kKeyMajor = true:  resident tiles K, V (this CTA's 128 keys), streamed Q, dO; accumulators dV, dK.
//                    TMEM lanes = keys, columns = queries: lse / delta vary along the columns.
// kKeyMajor = false: resident tiles Q, dO (this CTA's 128 queries), streamed K, V; accumulator dQ.
//                    TMEM lanes = queries, columns = keys: lse / delta are per thread.
template <bool kKeyMajor>
__global__ void __launch_bounds__(kBwd2Threads, 1)
attn_bwd2_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                 const __grid_constant__ Bwd2Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sR0 = smem;                      // resident: K (key-major) or Q
  uint8_t* sR1 = smem + kTile;              // resident: V (key-major) or dO
  uint8_t* sS0 = smem + 2 * kTile;          // ring of streamed tiles: Q or K
  uint8_t* sS1 = sS0 + kRing * kTile;       //                          dO or V
  uint64_t* bars = reinterpret_cast<uint64_t*>(sS1 + kRing * kTile);
  uint64_t* res_full = bars;
  uint64_t* ring_full = bars + 1;           // [kRing]
  uint64_t* ring_empty = bars + 3;          // [kRing]
  uint64_t* s_full = bars + 5;              // [2] (key-major uses [0] only)
  uint64_t* dp_full = bars + 7;
  uint64_t* p_ready = bars + 8;             // key-major: P^T is in TMEM
  uint64_t* ds_ready = bars + 9;            // dS is in TMEM
  uint64_t* acc_done = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = a.seq / kBlk;
  // same block order as the forward kernel: per group of batch-heads the longest tiles first (key block 0 / the
  // last query block stream the most)
  const int blk = kKeyMajor ? (int)blockIdx.y : (a.causal ? nblk - 1 - (int)blockIdx.y : (int)blockIdx.y);
  const int bh = blockIdx.z * gridDim.x + blockIdx.x;
  const int h = bh % a.heads, b = bh / a.heads;
  // streamed blocks: queries i0 .. nblk-1 for a key block, keys 0 .. blk for a query block
  const int i0 = kKeyMajor && a.causal ? blk : 0;
  const int n_it = kKeyMajor ? nblk - i0 : (a.causal ? blk + 1 : nblk);
  const int colq = h * 3 * kD;
  const uint64_t tmo = a.timeout_ns;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm_qkv);
    tma_prefetch_desc(&tm_do);
    mbar_init(res_full, 1);
    for (int i = 0; i < kRing; ++i) {
      mbar_init(ring_full + i, 1);
      mbar_init(ring_empty + i, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_full + 1, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, 256);
    mbar_init(ds_ready, 256);
    mbar_init(acc_done, 1);
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
  // key-major:   S^T [0,128)  dP^T [128,256)  dV [256,384)  dK [384,512)
  // query-major: S buffers [0,128) [128,256)  dP [256,384)  dQ [384,512)
  const uint32_t t_dp = tmem + (kKeyMajor ? 128 : 256);
  const uint32_t t_acc0 = tmem + (kKeyMajor ? 256 : 384), t_acc1 = tmem + 384;

  if (warp == 0) {
    if (lane == 0) {
      const int rrow = b * a.seq + blk * kBlk;
      mbar_expect_tx(res_full, 2 * kTile);
      if (kKeyMajor) {
        load_tile(sR0, &tm_qkv, res_full, colq + kD, rrow);        // K
        load_tile(sR1, &tm_qkv, res_full, colq + 2 * kD, rrow);    // V
      } else {
        load_tile(sR0, &tm_qkv, res_full, colq, rrow);             // Q
        load_tile(sR1, &tm_do, res_full, h * kD, rrow);            // dO
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it & 1;
        if (!mbar_wait(ring_empty + st, ((it >> 1) & 1) ^ 1, 6 * tmo)) {
          report(a.status, kErrAttn + 11, it, 0);
          break;
        }
        const int srow = b * a.seq + (i0 + it) * kBlk;
        mbar_expect_tx(ring_full + st, 2 * kTile);
        if (kKeyMajor) {
          load_tile(sS0 + st * kTile, &tm_qkv, ring_full + st, colq, srow);            // Q
          load_tile(sS1 + st * kTile, &tm_do, ring_full + st, h * kD, srow);           // dO
        } else {
          load_tile(sS0 + st * kTile, &tm_qkv, ring_full + st, colq + kD, srow);       // K
          load_tile(sS1 + st * kTile, &tm_qkv, ring_full + st, colq + 2 * kD, srow);   // V
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_s = make_idesc_bf16(128, 128, 0, 0);      // A K-major (smem) * B K-major
      const uint32_t id_g = make_idesc_bf16(128, 128, 0, 1);      // A (TMEM) * B MN-major
      // all operand descriptors, once: resident tiles; ring stage 0 (stage 1 = + kTile >> 4 in the
      // start-address field)
      uint64_t dr0[8], dr1[8], ds0k[8], ds1k[8], ds0m[8], ds1m[8];
      {
        const uint32_t r0 = smem_u32(sR0), r1 = smem_u32(sR1), b0 = smem_u32(sS0), b1 = smem_u32(sS1);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          dr0[k] = desc_kmajor(r0, k);
          dr1[k] = desc_kmajor(r1, k);
          ds0k[k] = desc_kmajor(b0, k);
          ds1k[k] = desc_kmajor(b1, k);
          ds0m[k] = desc_mnmajor(b0, k);
          ds1m[k] = desc_mnmajor(b1, k);
        }
      }
      constexpr uint64_t kStageOff = (uint64_t)(kTile >> 4);
      bool ok = mbar_wait(res_full, 0, 2 * tmo);
      if (!ok) report(a.status, kErrAttn + 12, 0, 0);
      auto wait_ring = [&](int it) -> bool {
        if (mbar_wait(ring_full + (it & 1), (it >> 1) & 1, 4 * tmo)) {
          tc_fence_after_sync();
          return true;
        }
        report(a.status, kErrAttn + 13, it, 0);
        return false;
      };
      auto wait_ew = [&](uint64_t* bar, int it, uint32_t code) -> bool {
        if (mbar_wait(bar, it & 1, 8 * tmo)) {
          tc_fence_after_sync();
          return true;
        }
        report(a.status, code, it, 0);
        return false;
      };
      // S (or S^T) of block `it` into score buffer `buf`; dP (or dP^T) of block `it`
      auto issue_s = [&](int it, int buf) {
        const uint64_t so = (it & 1) ? kStageOff : 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tmem + buf * 128, dr0[k], ds0k[k] + so, id_s, k != 0);
        umma_commit(s_full + buf);
      };
      auto issue_dp = [&](int it) {
        const uint64_t so = (it & 1) ? kStageOff : 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(t_dp, dr1[k], ds1k[k] + so, id_s, k != 0);
        umma_commit(dp_full);
      };
      if (ok && n_it > 0) {
        ok = wait_ring(0);
        if (ok) {
          issue_s(0, 0);
          issue_dp(0);
        }
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const uint64_t so = (it & 1) ? kStageOff : 0;
        const bool more = it + 1 < n_it;
        if (kKeyMajor) {
          if (!(ok = wait_ew(p_ready, it, kErrAttn + 14))) break;
#pragma unroll
          for (int k = 0; k < 8; ++k)   // dV += P^T dO   (contraction over the 128 queries)
            umma_f16_ts(t_acc0, tmem + (k >> 2) * 64 + (k & 3) * 8, ds1m[k] + so, id_g, (it | k) != 0);
          if (more) {
            if (!(ok = wait_ring(it + 1))) break;
            issue_s(it + 1, 0);         // S^T region: P^T(it) was read by the products just issued
          }
          if (!(ok = wait_ew(ds_ready, it, kErrAttn + 14))) break;
#pragma unroll
          for (int k = 0; k < 8; ++k)   // dK += dS^T Q
            umma_f16_ts(t_acc1, t_dp + (k >> 2) * 64 + (k & 3) * 8, ds0m[k] + so, id_g, (it | k) != 0);
          umma_commit(ring_empty + (it & 1));
          if (more) issue_dp(it + 1);
        } else {
          if (more) {
            if (!(ok = wait_ring(it + 1))) break;
            issue_s(it + 1, (it + 1) & 1);
          }
          if (!(ok = wait_ew(ds_ready, it, kErrAttn + 14))) break;
#pragma unroll
          for (int k = 0; k < 8; ++k)   // dQ += dS K     (contraction over the 128 keys)
            umma_f16_ts(t_acc0, t_dp + (k >> 2) * 64 + (k & 3) * 8, ds0m[k] + so, id_g, (it | k) != 0);
          umma_commit(ring_empty + (it & 1));
          if (more) issue_dp(it + 1);
        }
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;                     // which 64 of the 128 columns
    const int row = q4 * 32 + lane;                       // TMEM lane: key (key-major) or query
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    const float sl2 = a.scale * kLog2e;
    const int64_t stat0 = ((int64_t)b * a.heads + h) * a.seq;
    float my_lse2 = 0.f, my_delta = 0.f;
    if (!kKeyMajor) {
      my_lse2 = a.lse2[stat0 + blk * kBlk + row];
      my_delta = a.delta[stat0 + blk * kBlk + row];
    }
    const int me = blk * kBlk + row;                      // this lane's key (key-major) or query index
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int sb = kKeyMajor ? 0 : (it & 1);
      const uint32_t ts = tmem + lane_off + sb * 128 + half * 64;
      const uint32_t tdp = t_dp + lane_off + half * 64;
      const int c0 = (i0 + it) * kBlk + half * 64;        // first streamed index of this thread's columns
      // causal: a score survives when key <= query; only blocks that touch the diagonal pay for it
      const bool masked = a.causal && (kKeyMajor ? (c0 < me) : (c0 + 63 > me));
      uint32_t pk[32];                                    // P of this thread's 64 columns, packed bf16
      // ---- phase 1: P = exp2(S * scale * log2(e) - lse2) ----
      if (!warp_wait(s_full + sb, kKeyMajor ? (it & 1) : ((it >> 1) & 1), 8 * tmo)) {
        if (lane == 0) report(a.status, kErrAttn + 15, it, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32];
        tmem_ld_32x32(ts + c * 32, rs);
        float ls[32];
        if (kKeyMajor) {   // one address per warp: broadcast loads of 16 bytes
          const float4* lp = reinterpret_cast<const float4*>(a.lse2 + stat0 + c0 + c * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 x = __ldg(lp + i);
            ls[4 * i] = x.x; ls[4 * i + 1] = x.y; ls[4 * i + 2] = x.z; ls[4 * i + 3] = x.w;
          }
        }
        tmem_ld_wait();
        if (!masked) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = fast_exp2(fmaf(__uint_as_float(rs[i]), sl2, -(kKeyMajor ? ls[i] : my_lse2)));
            const float e1 = fast_exp2(fmaf(__uint_as_float(rs[i + 1]), sl2, -(kKeyMajor ? ls[i + 1] : my_lse2)));
            pk[c * 16 + (i >> 1)] = pack_bf16(e0, e1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float e0 = fast_exp2(fmaf(__uint_as_float(rs[i]), sl2, -(kKeyMajor ? ls[i] : my_lse2)));
            float e1 = fast_exp2(fmaf(__uint_as_float(rs[i + 1]), sl2, -(kKeyMajor ? ls[i + 1] : my_lse2)));
            const int q0 = c0 + c * 32 + i;
            if (!(kKeyMajor ? (me <= q0) : (q0 <= me))) e0 = 0.f;
            if (!(kKeyMajor ? (me <= q0 + 1) : (q0 + 1 <= me))) e1 = 0.f;
            pk[c * 16 + (i >> 1)] = pack_bf16(e0, e1);
          }
        }
      }
      if (kKeyMajor) {
        // P^T over this thread's own S^T columns: 64 bf16 = 32 TMEM columns from the half's first column
        uint32_t lo[16], hi[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) { lo[i] = pk[i]; hi[i] = pk[16 + i]; }
        tmem_st_32x16(ts, lo);
        tmem_st_32x16(ts + 16, hi);
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(p_ready);
      }
      // ---- phase 2: dS = P * (dP * scale - delta * scale) ----
      if (!warp_wait(dp_full, it & 1, 8 * tmo)) {
        if (lane == 0) report(a.status, kErrAttn + 16, it, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t dk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rp[32];
        tmem_ld_32x32(tdp + c * 32, rp);
        float dl[32];
        if (kKeyMajor) {
          const float4* dp = reinterpret_cast<const float4*>(a.delta + stat0 + c0 + c * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 y = __ldg(dp + i);
            dl[4 * i] = y.x; dl[4 * i + 1] = y.y; dl[4 * i + 2] = y.z; dl[4 * i + 3] = y.w;
          }
        }
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const uint32_t pp = pk[c * 16 + (i >> 1)];
          const float e0 = __uint_as_float(pp << 16), e1 = __uint_as_float(pp & 0xffff0000u);
          const float g0 = e0 * fmaf(__uint_as_float(rp[i]), a.scale, -(kKeyMajor ? dl[i] : my_delta));
          const float g1 = e1 * fmaf(__uint_as_float(rp[i + 1]), a.scale, -(kKeyMajor ? dl[i + 1] : my_delta));
          dk[c * 16 + (i >> 1)] = pack_bf16(g0, g1);
        }
      }
      {
        uint32_t lo[16], hi[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) { lo[i] = dk[i]; hi[i] = dk[16 + i]; }
        tmem_st_32x16(tdp, lo);       // dS over this thread's own dP columns
        tmem_st_32x16(tdp + 16, hi);
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(ds_ready);
      }
    }
    if (ok) {
      if (!warp_wait(acc_done, 0, 8 * tmo)) {
        if (lane == 0) report(a.status, kErrAttn + 17, 0, 0);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after_sync();
      // accumulators -> bf16 rows of dqkv; the two threads of a lane take 64 columns each
      __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(a.dqkv) +
                            ((int64_t)b * a.seq + blk * kBlk + row) * (a.heads * 3 * kD) + colq;
      const int n_acc = kKeyMajor ? 2 : 1;
#pragma unroll 1
      for (int which = 0; which < n_acc; ++which) {
        // key-major: acc0 = dV, acc1 = dK;  query-major: acc0 = dQ
        const uint32_t t = (which == 0 ? t_acc0 : t_acc1) + lane_off + half * 64;
        __nv_bfloat16* dst = base + (kKeyMajor ? (which == 0 ? 2 * kD : kD) : 0) + half * 64;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1]));
            v.y = pack_bf16(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
            v.z = pack_bf16(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]));
            v.w = pack_bf16(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = v;
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

// The shared-memory attribute is per device: set it once on every device that launches.
cudaError_t configure_device() {
  static bool configured[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && configured[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(attn_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwd2Smem);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(attn_bwd2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBwd2Smem);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(attn_bwd2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBwd2Smem);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64) configured[dev] = true;
  return cudaSuccess;
}

// Batch-heads per block-order group: the largest divisor of batch * heads that is at most 32.
int bh_group(int batch, int heads) {
  const int n = batch * heads;
  int g = 1;
  for (int d = 1; d <= 32; ++d)
    if (n % d == 0) g = d;
  return g;
}

}  // namespace

cudaError_t attention_fwd(const void* qkv, void* out, float* lse, int batch, int seq, int heads,
                          int causal, float scale, uint32_t* status, cudaStream_t stream) {
  if (seq % kBlk != 0 || batch <= 0 || heads <= 0 || (int64_t)batch * heads > 65535 || seq / kBlk > 65535)
    return cudaErrorInvalidValue;
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
  const int grp = bh_group(batch, heads);
  dim3 grid(grp, seq / kBlk, batch * heads / grp);
  attn_fwd2_kernel<<<grid, 192, kFwd2Smem, stream>>>(tm, a);
  return cudaGetLastError();
}

cudaError_t attention_bwd(const void* qkv, const void* out, const void* dout, const float* lse,
                          void* dqkv, float* dq_acc, float* delta, int batch, int seq, int heads,
                          int causal, float scale, uint32_t* status, cudaStream_t stream) {
  if (seq % kBlk != 0 || batch <= 0 || heads <= 0 || (int64_t)batch * heads > 65535 || seq / kBlk > 65535)
    return cudaErrorInvalidValue;
  {
    cudaError_t e0 = configure_device();
    if (e0 != cudaSuccess) return e0;
  }
  const int64_t tokens = (int64_t)batch * seq;
  {
    // delta * scale into `delta`, lse * log2(e) into the head of the `dq_acc` scratch
    const int64_t warps = tokens * heads;
    const int threads = 256;
    const int64_t blocks = (warps * 32 + threads - 1) / threads;
    attn_delta_kernel<<<(unsigned)blocks, threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout), delta, batch, seq, heads,
        lse, dq_acc, scale);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  CUtensorMap tq, td;
  const uint64_t width = (uint64_t)heads * 3 * kD, wdo = (uint64_t)heads * kD;
  if (make_tensor_map_2d(&tq, qkv, width, (uint64_t)tokens, width * 2, 64, kBlk) != 0) return cudaErrorInvalidValue;
  if (make_tensor_map_2d(&td, dout, wdo, (uint64_t)tokens, wdo * 2, 64, kBlk) != 0) return cudaErrorInvalidValue;
  // two deterministic kernels: dK / dV per key block, dQ per query block
  Bwd2Args g{};
  g.dqkv = dqkv;
  g.lse2 = dq_acc;     // lse * log2(e)
  g.delta = delta;     // delta * scale
  g.batch = batch; g.seq = seq; g.heads = heads; g.causal = causal;
  g.scale = scale;
  g.status = status;
  g.timeout_ns = 2000000000ull;
  const int grp = bh_group(batch, heads);
  dim3 grid2(grp, seq / kBlk, batch * heads / grp);
  attn_bwd2_kernel<true><<<grid2, kBwd2Threads, kBwd2Smem, stream>>>(tq, td, g);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  attn_bwd2_kernel<false><<<grid2, kBwd2Threads, kBwd2Smem, stream>>>(tq, td, g);
  return cudaGetLastError();
}

}  // namespace msb
