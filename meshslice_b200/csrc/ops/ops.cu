// Memory-bound kernels of the GPT block: LayerNorm (+ residual) over column-sharded features,
// GeLU, AdamW, vocab-parallel cross-entropy, embedding, gradient norm.  All of them stream
// 16-byte vectors (8 bf16) and keep statistics in fp32.
#include "ops.h"

#include <cuda_bf16.h>
#include <string.h>

namespace msb {

namespace {

constexpr int kLnThreads = 256;
constexpr int kLnBwdThreads = 512;
constexpr int kLnGroupedMaxCols = 2048;   // rows up to this width run several per CTA in ln_bwd_kernel

// ---- cross-GPU row exchange (see RowExchange in ops.h) ----
__device__ __forceinline__ void ex_red_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ex_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ex_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Thread 0 of the CTA publishes "this CTA's rows are written" on every peer.
__device__ __forceinline__ void ex_signal(const RowExchange& ex) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int p = 0; p < ex.n; ++p)
      if (p != ex.me) ex_red_release_sys(ex.counter[p], 1u);
  }
}
// All threads return true once every CTA of every peer has published; false after the deadline
// (the status word then says which kernel gave up: code 20 + kind).
__device__ __forceinline__ bool ex_wait(const RowExchange& ex, uint32_t kind) {
  int ok = 1;
  if (threadIdx.x == 0) {
    const uint64_t t0 = ex_timer_ns();
    uint32_t it = 0;
    while ((int32_t)(ex_ld_acquire_sys(ex.my_counter) - ex.target) < 0) {
      if ((++it & 0xf) == 0) {
        if (ex_timer_ns() - t0 > ex.timeout_ns) {
          ok = 0;
          if (atomicCAS(ex.status, 0u, 20u + kind) == 0u) {
            ex.status[1] = blockIdx.x;
            ex.status[2] = ex_ld_acquire_sys(ex.my_counter);
            ex.status[3] = ex.target;
          }
          break;
        }
        __nanosleep(128);
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}
// Writes this GPU's W-float contribution of one row into its slot on every GPU of the group.
template <int W>
__device__ __forceinline__ void ex_put(const RowExchange& ex, int row, const float (&v)[W]) {
  for (int p = 0; p < ex.n; ++p) {
    float* d = ex.dst[p] + (int64_t)row * W;
#pragma unroll
    for (int i = 0; i < W; ++i) d[i] = v[i];
  }
}
// Source q's contribution of one row (L1 bypassed: peers wrote it).
__device__ __forceinline__ float ex_get(const RowExchange& ex, int q, int row, int width, int i) {
  return __ldcg(ex.slots + q * ex.stride + (int64_t)row * width + i);
}

__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  f[0] = bf_lo(u.x); f[1] = bf_hi(u.x); f[2] = bf_lo(u.y); f[3] = bf_hi(u.y);
  f[4] = bf_lo(u.z); f[5] = bf_hi(u.z); f[6] = bf_lo(u.w); f[7] = bf_hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack2(f[0], f[1]); u.y = pack2(f[2], f[3]); u.z = pack2(f[4], f[5]); u.w = pack2(f[6], f[7]);
  return u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum of two values over the CTA; every thread gets the result.  `red` holds 2 * 32 floats.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) { red[w] = a; red[32 + w] = b; }
  __syncthreads();
  a = l < nw ? red[l] : 0.f;
  b = l < nw ? red[32 + l] : 0.f;
  a = warp_sum(a);
  b = warp_sum(b);
}
__device__ __forceinline__ float block_max(float a, float* red) {
  a = warp_max(a);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = a;
  __syncthreads();
  a = l < nw ? red[l] : -INFINITY;
  return warp_max(a);
}

__device__ __forceinline__ float gelu_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u = k0 * (x + k1 * x * x * x);
  const float t = tanhf(u);
  const float du = k0 * (1.0f + 3.0f * k1 * x * x);
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
}

// ------------------------------------------------------------------------------------------
// LayerNorm forward.  One CTA per row (grid-stride), row cached in registers.
// ------------------------------------------------------------------------------------------
template <int MAXV>
__global__ void __launch_bounds__(kLnThreads)
ln_fwd_kernel(int mode, const uint4* __restrict__ x, const uint4* __restrict__ res,
              uint4* __restrict__ h_out, uint4* __restrict__ y, const uint4* __restrict__ gamma,
              const uint4* __restrict__ beta, float* __restrict__ stats,
              float* __restrict__ mean_rstd, int rows, int cols, int total_cols, float eps,
              const __grid_constant__ RowExchange ex) {
  __shared__ float red[64];
  const int nvec = cols >> 3;
  // With an exchange (ex.n > 0) mode 1 writes the partial statistics of its rows to every GPU of
  // the mesh row and counts one arrival per CTA on every peer; mode 2 first waits (bounded) for
  // the arrivals of all peers' CTAs and then sums the sources' statistics in fixed order.
  const bool exchange = ex.n > 0;
  if (exchange && mode == 2 && !ex_wait(ex, 0u)) return;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float vals[MAXV][8];
    float s = 0.f, ss = 0.f;
    const int64_t base = (int64_t)row * nvec;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int v = threadIdx.x + k * blockDim.x;
      if (v < nvec) {
        unpack8(x[base + v], vals[k]);
        if (mode != 2 && res != nullptr) {
          float r[8];
          unpack8(res[base + v], r);
#pragma unroll
          for (int i = 0; i < 8; ++i) vals[k][i] += r[i];
        }
        if (mode != 2 && h_out != nullptr) {
          const uint4 hp = pack8(vals[k]);
          h_out[base + v] = hp;
          unpack8(hp, vals[k]);  // statistics of the rounded values the backward pass sees
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) { s += vals[k][i]; ss += vals[k][i] * vals[k][i]; }
      }
    }
    float mean, rstd;
    if (mode == 2) {
      if (exchange) {
        s = 0.f;
        ss = 0.f;
        for (int q = 0; q < ex.n; ++q) { s += ex_get(ex, q, row, 2, 0); ss += ex_get(ex, q, row, 2, 1); }
      } else {
        s = stats[2 * row];
        ss = stats[2 * row + 1];
      }
    } else {
      block_sum2(s, ss, red);
      if (mode == 1) {
        if (threadIdx.x == 0) {
          if (exchange) {
            const float v2[2] = {s, ss};
            ex_put<2>(ex, row, v2);
          } else {
            stats[2 * row] = s;
            stats[2 * row + 1] = ss;
          }
        }
        continue;
      }
    }
    mean = s / (float)total_cols;
    rstd = rsqrtf(fmaxf(ss / (float)total_cols - mean * mean, 0.f) + eps);
    if (threadIdx.x == 0 && mean_rstd != nullptr) {
      mean_rstd[2 * row] = mean;
      mean_rstd[2 * row + 1] = rstd;
    }
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int v = threadIdx.x + k * blockDim.x;
      if (v < nvec) {
        float g[8], b[8], o[8];
        if (gamma != nullptr) unpack8(gamma[v], g);
        if (beta != nullptr) unpack8(beta[v], b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float t = (vals[k][i] - mean) * rstd;
          if (gamma != nullptr) t *= g[i];
          if (beta != nullptr) t += b[i];
          o[i] = t;
        }
        y[base + v] = pack8(o);
      }
    }
  }
  if (exchange && mode == 1) ex_signal(ex);
}

// ------------------------------------------------------------------------------------------
// LayerNorm backward
// ------------------------------------------------------------------------------------------
// Sum of two values over the `gw` consecutive warps that share a row; every thread of the group gets the result.
__device__ __forceinline__ void group_sum2(float& a, float& b, float* red, int gw) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) { red[w] = a; red[32 + w] = b; }
  __syncthreads();
  const int w0 = w / gw * gw;
  a = 0.f;
  b = 0.f;
  for (int i = 0; i < gw; ++i) { a += red[w0 + i]; b += red[32 + w0 + i]; }
}

// A CTA of up to kLnBwdThreads threads walks the rows grid-stride.  A 4096-wide row is one 16-byte vector per
// thread: the per-thread dgamma / dbeta accumulators (16 registers per vector) are what limits occupancy, and all
// three input vectors of a row (dy, h, dres) are requested before anything waits for them.  The rows stay packed
// in registers between the two passes; gamma is loaded once per CTA.
// GROUPED (rows of at most 256 vectors, e.g. column shards): the CTA works on blockDim.x / tpr rows at a time,
// `tpr` threads (whole warps) per row, and adds the row groups' dgamma / dbeta in shared memory before its one
// atomic per column, so that narrow rows neither idle most of a CTA nor multiply the atomics.
template <int MAXV, bool GROUPED>
__global__ void __launch_bounds__(kLnBwdThreads, MAXV == 1 ? 2 : 1)
ln_bwd_kernel(int mode, const uint4* __restrict__ dy, const uint4* __restrict__ h,
              const uint4* __restrict__ gamma, const float* __restrict__ mean_rstd,
              const uint4* __restrict__ dres, uint4* __restrict__ dx, float* __restrict__ stats,
              float* __restrict__ dgamma, float* __restrict__ dbeta, int rows, int cols,
              int total_cols, int tpr_arg, const __grid_constant__ RowExchange ex) {
  static_assert(!GROUPED || MAXV == 1, "grouped rows are one vector per thread");
  __shared__ float red[64];
  __shared__ float comb[GROUPED ? 2 * kLnGroupedMaxCols : 1];
  const int nvec = cols >> 3;
  const int tpr = GROUPED ? tpr_arg : (int)blockDim.x;            // threads per row
  const int sub = GROUPED ? (int)threadIdx.x / tpr : 0;           // which of the CTA's rows
  const int tx = GROUPED ? (int)threadIdx.x - sub * tpr : (int)threadIdx.x;
  const int rows_per_cta = GROUPED ? (int)blockDim.x / tpr : 1;
  float accg[MAXV][8], accb[MAXV][8];
  uint4 pg[MAXV];
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
#pragma unroll
    for (int i = 0; i < 8; ++i) { accg[k][i] = 0.f; accb[k][i] = 0.f; }
    const int v = tx + k * tpr;
    pg[k] = (gamma != nullptr && v < nvec) ? gamma[v] : make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
  }
  // exchange of the partial sums with the GPUs of the mesh row: see ln_fwd_kernel
  const bool exchange = ex.n > 0;
  if (exchange && mode == 2 && !ex_wait(ex, 1u)) return;
  const bool want_param_grads = mode != 2 && dgamma != nullptr;
  const bool want_dres = mode != 1 && dres != nullptr;

  for (int r0 = blockIdx.x * rows_per_cta; r0 < rows; r0 += gridDim.x * rows_per_cta) {
    const int row = r0 + sub;
    const bool live = row < rows;          // the last rows of a grouped CTA may be missing; barriers stay uniform
    const int64_t base = (int64_t)row * nvec;
    uint4 pd[MAXV], ph[MAXV], pr[MAXV];
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int v = tx + k * tpr;
      pd[k] = make_uint4(0u, 0u, 0u, 0u);
      ph[k] = make_uint4(0u, 0u, 0u, 0u);
      if (live && v < nvec) {
        pd[k] = __ldcs(dy + base + v);
        ph[k] = __ldcs(h + base + v);
        if (want_dres) pr[k] = __ldcs(dres + base + v);
      }
    }
    const float mean = live ? mean_rstd[2 * row] : 0.f, rstd = live ? mean_rstd[2 * row + 1] : 0.f;
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int v = tx + k * tpr;
      if (live && v < nvec) {
        float d[8], hv[8], gm[8];
        unpack8(pd[k], d);
        unpack8(ph[k], hv);
        unpack8(pg[k], gm);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xh = (hv[i] - mean) * rstd;
          const float g = d[i] * gm[i];
          s1 += g;
          s2 += g * xh;
          if (want_param_grads) { accg[k][i] += d[i] * xh; accb[k][i] += d[i]; }
        }
      }
    }
    if (mode == 2) {
      if (live) {
        if (exchange) {
          s1 = 0.f;
          s2 = 0.f;
          for (int q = 0; q < ex.n; ++q) { s1 += ex_get(ex, q, row, 2, 0); s2 += ex_get(ex, q, row, 2, 1); }
        } else {
          s1 = stats[2 * row];
          s2 = stats[2 * row + 1];
        }
      }
    } else {
      if (GROUPED) group_sum2(s1, s2, red, tpr >> 5);
      else block_sum2(s1, s2, red);
      if (mode == 1) {
        if (tx == 0 && live) {
          if (exchange) {
            const float v2[2] = {s1, s2};
            ex_put<2>(ex, row, v2);
          } else {
            stats[2 * row] = s1;
            stats[2 * row + 1] = s2;
          }
        }
        continue;
      }
    }
    const float m1 = s1 / (float)total_cols, m2 = s2 / (float)total_cols;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int v = tx + k * tpr;
      if (live && v < nvec) {
        float d[8], hv[8], gm[8], o[8];
        unpack8(pd[k], d);
        unpack8(ph[k], hv);
        unpack8(pg[k], gm);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (d[i] * gm[i] - m1 - (hv[i] - mean) * rstd * m2);
        if (want_dres) {
          float r[8];
          unpack8(pr[k], r);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += r[i];
        }
        __stcs(dx + base + v, pack8(o));
      }
    }
  }
  if (exchange && mode == 1) ex_signal(ex);
  if (want_param_grads) {
    if (GROUPED) {
      for (int i = threadIdx.x; i < 2 * cols; i += blockDim.x) comb[i] = 0.f;
      __syncthreads();
      if (tx < nvec) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          atomicAdd(comb + tx * 8 + i, accg[0][i]);
          atomicAdd(comb + cols + tx * 8 + i, accb[0][i]);
        }
      }
      __syncthreads();
      for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        atomicAdd(dgamma + i, comb[i]);
        if (dbeta != nullptr) atomicAdd(dbeta + i, comb[cols + i]);
      }
    } else {
#pragma unroll
      for (int k = 0; k < MAXV; ++k) {
        const int v = tx + k * tpr;
        if (v < nvec) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            atomicAdd(dgamma + v * 8 + i, accg[k][i]);
            if (dbeta != nullptr) atomicAdd(dbeta + v * 8 + i, accb[k][i]);
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// elementwise
// ------------------------------------------------------------------------------------------
__global__ void gelu_fwd_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int64_t nvec) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(x[i], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = gelu_f(f[k]);
    y[i] = pack8(f);
  }
}
__global__ void gelu_bwd_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ x,
                                uint4* __restrict__ dx, int64_t nvec) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    float f[8], d[8];
    unpack8(x[i], f);
    unpack8(dy[i], d);
#pragma unroll
    for (int k = 0; k < 8; ++k) d[k] *= gelu_grad_f(f[k]);
    dx[i] = pack8(d);
  }
}
__global__ void add_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b,
                           uint4* __restrict__ o, int64_t nvec) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    float f[8], g[8];
    unpack8(a[i], f);
    unpack8(b[i], g);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] += g[k];
    o[i] = pack8(f);
  }
}
__global__ void cast_kernel(const float4* __restrict__ in, uint2* __restrict__ out, int64_t nvec,
                            int accumulate) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    float4 f = in[i];
    if (accumulate) {
      const uint2 c = out[i];
      f.x += bf_lo(c.x); f.y += bf_hi(c.x); f.z += bf_lo(c.y); f.w += bf_hi(c.y);
    }
    uint2 o;
    o.x = pack2(f.x, f.y);
    o.y = pack2(f.z, f.w);
    out[i] = o;
  }
}

// ------------------------------------------------------------------------------------------
// AdamW: 4 elements per thread
// ------------------------------------------------------------------------------------------
__global__ void adamw_kernel(uint2* __restrict__ param, float4* __restrict__ master,
                             float4* __restrict__ m, float4* __restrict__ v,
                             const void* __restrict__ grad, int grad_fp32, int64_t nvec, float lr,
                             float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                             const float* __restrict__ grad_scale) {
  const float gs = grad_scale != nullptr ? *grad_scale : 1.0f;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    float g[4];
    if (grad_fp32) {
      const float4 gg = reinterpret_cast<const float4*>(grad)[i];
      g[0] = gg.x; g[1] = gg.y; g[2] = gg.z; g[3] = gg.w;
    } else {
      const uint2 gg = reinterpret_cast<const uint2*>(grad)[i];
      g[0] = bf_lo(gg.x); g[1] = bf_hi(gg.x); g[2] = bf_lo(gg.y); g[3] = bf_hi(gg.y);
    }
    float4 p4 = master[i], m4 = m[i], v4 = v[i];
    float p[4] = {p4.x, p4.y, p4.z, p4.w};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = g[k] * gs;
      mm[k] = beta1 * mm[k] + (1.f - beta1) * gk;
      vv[k] = beta2 * vv[k] + (1.f - beta2) * gk * gk;
      const float mh = mm[k] / bc1, vh = vv[k] / bc2;
      p[k] = p[k] - lr * (mh / (sqrtf(vh) + eps) + wd * p[k]);
    }
    master[i] = make_float4(p[0], p[1], p[2], p[3]);
    m[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    v[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    uint2 o;
    o.x = pack2(p[0], p[1]);
    o.y = pack2(p[2], p[3]);
    param[i] = o;
  }
}

__global__ void sumsq_kernel(const void* __restrict__ x, int is_fp32, int64_t nvec,
                             float* __restrict__ out) {
  __shared__ float red[64];
  float s = 0.f, dummy = 0.f;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    if (is_fp32) {
      const float4 g = reinterpret_cast<const float4*>(x)[i];
      s += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
    } else {
      const uint2 g = reinterpret_cast<const uint2*>(x)[i];
      const float a = bf_lo(g.x), b = bf_hi(g.x), c = bf_lo(g.y), d = bf_hi(g.y);
      s += a * a + b * b + c * c + d * d;
    }
  }
  block_sum2(s, dummy, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// ------------------------------------------------------------------------------------------
// vocab-parallel cross-entropy: one CTA per row
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
ce_partial_kernel(const __nv_bfloat16* __restrict__ logits, int64_t ld,
                  const int64_t* __restrict__ targets, int rows, int cols, int col_offset,
                  int vocab, float* __restrict__ row_max, float* __restrict__ row_sumexp,
                  float* __restrict__ tgt_logit, const __grid_constant__ RowExchange ex) {
  __shared__ float red[64];
  const int valid = max(0, min(cols, vocab - col_offset));
  const int nvec = valid >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* p = logits + (int64_t)row * ld;
    const uint4* pv = reinterpret_cast<const uint4*>(p);
    float mx = -INFINITY;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      unpack8(pv[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = fmaxf(mx, f[i]);
    }
    for (int c = nvec * 8 + threadIdx.x; c < valid; c += blockDim.x)
      mx = fmaxf(mx, __bfloat162float(p[c]));
    mx = block_max(mx, red);
    float s = 0.f, dummy = 0.f;
    if (valid > 0) {
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float f[8];
        unpack8(pv[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += __expf(f[i] - mx);
      }
      for (int c = nvec * 8 + threadIdx.x; c < valid; c += blockDim.x)
        s += __expf(__bfloat162float(p[c]) - mx);
    }
    block_sum2(s, dummy, red);
    if (threadIdx.x == 0) {
      const int64_t t = targets[row] - col_offset;
      const float tl = (t >= 0 && t < valid) ? __bfloat162float(p[t]) : 0.f;
      if (ex.n > 0) {        // publish (max, sum-exp relative to it, target logit) to the mesh row
        const float v3[3] = {mx, s, tl};
        ex_put<3>(ex, row, v3);
      } else {
        row_max[row] = mx;
        row_sumexp[row] = s;
        tgt_logit[row] = tl;
      }
    }
  }
  if (ex.n > 0) ex_signal(ex);
}

__global__ void __launch_bounds__(256)
ce_grad_kernel(__nv_bfloat16* __restrict__ logits, int64_t ld, const int64_t* __restrict__ targets,
               int rows, int cols, int col_offset, int vocab, const float* __restrict__ gmax,
               const float* __restrict__ gsumexp, float scale, float* __restrict__ row_loss,
               const __grid_constant__ RowExchange ex) {
  const int nvec = cols >> 3;
  if (ex.n > 0 && !ex_wait(ex, 2u)) return;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    __nv_bfloat16* p = logits + (int64_t)row * ld;
    uint4* pv = reinterpret_cast<uint4*>(p);
    float mx, se;
    if (ex.n > 0) {
      // combine the vocabulary slices of the mesh row in fixed order: global max, sum of the
      // rescaled partial sums, the one non-zero target logit; every GPU of the row gets the same
      mx = -INFINITY;
      for (int q = 0; q < ex.n; ++q) mx = fmaxf(mx, ex_get(ex, q, row, 3, 0));
      se = 0.f;
      float tl = 0.f;
      for (int q = 0; q < ex.n; ++q) {
        const float sq = ex_get(ex, q, row, 3, 1);
        if (sq > 0.f) se += sq * __expf(ex_get(ex, q, row, 3, 0) - mx);
        tl += ex_get(ex, q, row, 3, 2);
      }
      if (threadIdx.x == 0 && row_loss != nullptr) row_loss[row] = __logf(se) + mx - tl;
    } else {
      mx = gmax[row];
      se = gsumexp[row];
    }
    const float inv = scale / se;
    const int64_t t = targets[row] - col_offset;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      unpack8(pv[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = v * 8 + i;
        float gsm = (c + col_offset < vocab) ? __expf(f[i] - mx) * inv : 0.f;
        if (c == t) gsm -= scale;
        f[i] = gsm;
      }
      pv[v] = pack8(f);
    }
  }
}

// ------------------------------------------------------------------------------------------
// embedding
// ------------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ tokens,
                                     const uint4* __restrict__ tok_table,
                                     const uint4* __restrict__ pos_table, uint4* __restrict__ out,
                                     int n_tokens, int seq, int nvec) {
  for (int t = blockIdx.x; t < n_tokens; t += gridDim.x) {
    const int64_t tok = tokens[t];
    const int pos = t % seq;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float a[8], b[8];
      unpack8(tok_table[tok * nvec + v], a);
      unpack8(pos_table[(int64_t)pos * nvec + v], b);
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] += b[i];
      out[(int64_t)t * nvec + v] = pack8(a);
    }
  }
}
// token table: scatter-add with fp32 vector atomics; position table: plain sum over the batch
__global__ void embedding_bwd_tok_kernel(const int64_t* __restrict__ tokens,
                                         const uint4* __restrict__ dout, float* __restrict__ dtok,
                                         int n_tokens, int nvec) {
  for (int t = blockIdx.x; t < n_tokens; t += gridDim.x) {
    const int64_t tok = tokens[t];
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float a[8];
      unpack8(dout[(int64_t)t * nvec + v], a);
      float4* dst = reinterpret_cast<float4*>(dtok + (tok * nvec + v) * 8);
      atomicAdd(dst, make_float4(a[0], a[1], a[2], a[3]));
      atomicAdd(dst + 1, make_float4(a[4], a[5], a[6], a[7]));
    }
  }
}
__global__ void embedding_bwd_pos_kernel(const uint4* __restrict__ dout, float* __restrict__ dpos,
                                         int n_tokens, int seq, int nvec) {
  const int64_t total = (int64_t)seq * nvec;
  const int nb = n_tokens / seq;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t pos = i / nvec, v = i - pos * nvec;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int b = 0; b < nb; ++b) {
      float a[8];
      unpack8(dout[((int64_t)b * seq + pos) * nvec + v], a);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += a[k];
    }
    float* dst = dpos + i * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) dst[k] += acc[k];
  }
}

// One CTA per row: as many threads as the row has 16-byte vectors (64..256), so that short
// column-sharded rows do not leave half of the CTA idle.
inline int ln_threads(int cols) {
  const int nvec = cols / 8;
  int t = (nvec + 31) / 32 * 32;
  if (t < 64) t = 64;
  if (t > kLnThreads) t = kLnThreads;
  return t;
}

// Launch shape of ln_bwd_kernel for a local width: threads per CTA, threads per row, rows per CTA, vectors per thread.
struct LnBwdShape { int threads, tpr, rows_per_cta, maxv; };
inline LnBwdShape ln_bwd_shape(int cols) {
  const int nvec = cols / 8;
  int tpr = (nvec + 31) / 32 * 32;
  if (tpr < 32) tpr = 32;
  if (cols <= kLnGroupedMaxCols) {
    const int g = kLnBwdThreads / tpr;
    return {g * tpr, tpr, g, 1};
  }
  if (tpr > kLnBwdThreads) tpr = kLnBwdThreads;
  return {tpr, tpr, 1, (nvec + tpr - 1) / tpr};
}

inline int grid_for(int64_t n, int threads, int cap = 148 * 16) {
  int64_t g = (n + threads - 1) / threads;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace

// ------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------
int ce_grid(int rows) { return rows < 148 * 8 ? rows : 148 * 8; }

int ln_grid(int backward, int rows, int cols) {
  int cap = 148 * 16;
  if (backward) {
    // one resident wave (1024 threads per SM at 64 registers): every CTA ends with one atomic per column for
    // dgamma / dbeta, so CTAs beyond what is resident only add atomics
    const LnBwdShape sh = ln_bwd_shape(cols > 0 ? cols : 8 * kLnBwdThreads);
    cap = 148 * (1024 / sh.threads);
    const int groups = (rows + sh.rows_per_cta - 1) / sh.rows_per_cta;
    return groups < cap ? groups : cap;
  }
  return rows < cap ? rows : cap;
}

cudaError_t ln_fwd(int mode, const void* x, const void* res, void* h_out, void* y,
                   const void* gamma, const void* beta, float* stats, float* mean_rstd, int rows,
                   int cols, int total_cols, float eps, cudaStream_t stream, const RowExchange* exch) {
  if (cols % 8 != 0 || cols > 8 * kLnThreads * 8) return cudaErrorInvalidValue;
  if (exch != nullptr && mode != 1 && mode != 2) return cudaErrorInvalidValue;
  const int grid = ln_grid(0, rows, cols);
  RowExchange ex;
  if (exch != nullptr) ex = *exch; else memset(&ex, 0, sizeof(ex));
  auto X = reinterpret_cast<const uint4*>(x);
  auto R = reinterpret_cast<const uint4*>(res);
  auto H = reinterpret_cast<uint4*>(h_out);
  auto Y = reinterpret_cast<uint4*>(y);
  auto G = reinterpret_cast<const uint4*>(gamma);
  auto B = reinterpret_cast<const uint4*>(beta);
  const int threads = ln_threads(cols);
  const int nvec_per_thread = (cols / 8 + threads - 1) / threads;
  if (nvec_per_thread <= 1)
    ln_fwd_kernel<1><<<grid, threads, 0, stream>>>(mode, X, R, H, Y, G, B, stats, mean_rstd, rows, cols, total_cols, eps, ex);
  else if (nvec_per_thread <= 2)
    ln_fwd_kernel<2><<<grid, threads, 0, stream>>>(mode, X, R, H, Y, G, B, stats, mean_rstd, rows, cols, total_cols, eps, ex);
  else if (nvec_per_thread <= 4)
    ln_fwd_kernel<4><<<grid, threads, 0, stream>>>(mode, X, R, H, Y, G, B, stats, mean_rstd, rows, cols, total_cols, eps, ex);
  else
    ln_fwd_kernel<8><<<grid, threads, 0, stream>>>(mode, X, R, H, Y, G, B, stats, mean_rstd, rows, cols, total_cols, eps, ex);
  return cudaGetLastError();
}

cudaError_t ln_bwd(int mode, const void* dy, const void* h, const void* gamma,
                   const float* mean_rstd, const void* dres, void* dx, float* stats, float* dgamma,
                   float* dbeta, int rows, int cols, int total_cols, cudaStream_t stream,
                   const RowExchange* exch) {
  if (cols % 8 != 0 || cols > 8 * kLnBwdThreads * 4) return cudaErrorInvalidValue;
  if (exch != nullptr && mode != 1 && mode != 2) return cudaErrorInvalidValue;
  const int grid = ln_grid(1, rows, cols);
  RowExchange ex;
  if (exch != nullptr) ex = *exch; else memset(&ex, 0, sizeof(ex));
  auto DY = reinterpret_cast<const uint4*>(dy);
  auto H = reinterpret_cast<const uint4*>(h);
  auto G = reinterpret_cast<const uint4*>(gamma);
  auto DR = reinterpret_cast<const uint4*>(dres);
  auto DX = reinterpret_cast<uint4*>(dx);
  const LnBwdShape sh = ln_bwd_shape(cols);
  if (sh.rows_per_cta > 1 || cols <= kLnGroupedMaxCols)
    ln_bwd_kernel<1, true><<<grid, sh.threads, 0, stream>>>(mode, DY, H, G, mean_rstd, DR, DX, stats, dgamma, dbeta, rows, cols, total_cols, sh.tpr, ex);
  else if (sh.maxv <= 1)
    ln_bwd_kernel<1, false><<<grid, sh.threads, 0, stream>>>(mode, DY, H, G, mean_rstd, DR, DX, stats, dgamma, dbeta, rows, cols, total_cols, sh.tpr, ex);
  else if (sh.maxv <= 2)
    ln_bwd_kernel<2, false><<<grid, sh.threads, 0, stream>>>(mode, DY, H, G, mean_rstd, DR, DX, stats, dgamma, dbeta, rows, cols, total_cols, sh.tpr, ex);
  else
    ln_bwd_kernel<4, false><<<grid, sh.threads, 0, stream>>>(mode, DY, H, G, mean_rstd, DR, DX, stats, dgamma, dbeta, rows, cols, total_cols, sh.tpr, ex);
  return cudaGetLastError();
}

cudaError_t gelu_fwd(const void* x, void* y, int64_t n, cudaStream_t stream) {
  if (n % 8) return cudaErrorInvalidValue;
  gelu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(reinterpret_cast<const uint4*>(x), reinterpret_cast<uint4*>(y), n / 8);
  return cudaGetLastError();
}
cudaError_t gelu_bwd(const void* dy, const void* x, void* dx, int64_t n, cudaStream_t stream) {
  if (n % 8) return cudaErrorInvalidValue;
  gelu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(reinterpret_cast<const uint4*>(dy), reinterpret_cast<const uint4*>(x), reinterpret_cast<uint4*>(dx), n / 8);
  return cudaGetLastError();
}
cudaError_t add_bf16(const void* a, const void* b, void* out, int64_t n, cudaStream_t stream) {
  if (n % 8) return cudaErrorInvalidValue;
  add_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(reinterpret_cast<const uint4*>(a), reinterpret_cast<const uint4*>(b), reinterpret_cast<uint4*>(out), n / 8);
  return cudaGetLastError();
}
cudaError_t cast_f32_to_bf16(const float* in, void* out, int64_t n, int accumulate, cudaStream_t stream) {
  if (n % 4) return cudaErrorInvalidValue;
  cast_kernel<<<grid_for(n / 4, 256), 256, 0, stream>>>(reinterpret_cast<const float4*>(in), reinterpret_cast<uint2*>(out), n / 4, accumulate);
  return cudaGetLastError();
}

cudaError_t adamw_step(void* param, float* master, float* m, float* v, const void* grad,
                       int grad_fp32, int64_t n, float lr, float beta1, float beta2, float eps,
                       float weight_decay, float bias_corr1, float bias_corr2,
                       const float* grad_scale, cudaStream_t stream) {
  if (n % 4) return cudaErrorInvalidValue;
  adamw_kernel<<<grid_for(n / 4, 256), 256, 0, stream>>>(
      reinterpret_cast<uint2*>(param), reinterpret_cast<float4*>(master), reinterpret_cast<float4*>(m),
      reinterpret_cast<float4*>(v), grad, grad_fp32, n / 4, lr, beta1, beta2, eps, weight_decay,
      bias_corr1, bias_corr2, grad_scale);
  return cudaGetLastError();
}

cudaError_t sumsq(const void* x, int is_fp32, int64_t n, float* out, cudaStream_t stream) {
  if (n % 4) return cudaErrorInvalidValue;
  sumsq_kernel<<<grid_for(n / 4, 256, 148 * 8), 256, 0, stream>>>(x, is_fp32, n / 4, out);
  return cudaGetLastError();
}

cudaError_t ce_partial(const void* logits, int64_t ld, const int64_t* targets, int rows, int cols,
                       int col_offset, int vocab, float* row_max, float* row_sumexp,
                       float* tgt_logit, cudaStream_t stream, const RowExchange* exch) {
  RowExchange ex;
  if (exch != nullptr) ex = *exch; else memset(&ex, 0, sizeof(ex));
  if (ld % 8) return cudaErrorInvalidValue;
  const int grid = ce_grid(rows);
  ce_partial_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, targets, rows, cols, col_offset, vocab, row_max, row_sumexp, tgt_logit, ex);
  return cudaGetLastError();
}
cudaError_t ce_grad(void* logits, int64_t ld, const int64_t* targets, int rows, int cols,
                    int col_offset, int vocab, const float* gmax, const float* gsumexp, float scale,
                    cudaStream_t stream, float* row_loss, const RowExchange* exch) {
  RowExchange ex;
  if (exch != nullptr) ex = *exch; else memset(&ex, 0, sizeof(ex));
  if (ld % 8 || cols % 8) return cudaErrorInvalidValue;
  const int grid = ce_grid(rows);
  ce_grad_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(logits), ld, targets, rows, cols, col_offset, vocab, gmax, gsumexp, scale, row_loss, ex);
  return cudaGetLastError();
}

cudaError_t embedding_fwd(const int64_t* tokens, const void* tok_table, const void* pos_table,
                          void* out, int n_tokens, int seq, int cols, cudaStream_t stream) {
  if (cols % 8) return cudaErrorInvalidValue;
  const int grid = n_tokens < 148 * 16 ? n_tokens : 148 * 16;
  embedding_fwd_kernel<<<grid, 128, 0, stream>>>(tokens, reinterpret_cast<const uint4*>(tok_table), reinterpret_cast<const uint4*>(pos_table), reinterpret_cast<uint4*>(out), n_tokens, seq, cols / 8);
  return cudaGetLastError();
}
cudaError_t embedding_bwd(const int64_t* tokens, const void* dout, float* dtok, float* dpos,
                          int n_tokens, int seq, int cols, cudaStream_t stream) {
  if (cols % 8 || n_tokens % seq) return cudaErrorInvalidValue;
  const int grid = n_tokens < 148 * 16 ? n_tokens : 148 * 16;
  embedding_bwd_tok_kernel<<<grid, 128, 0, stream>>>(tokens, reinterpret_cast<const uint4*>(dout), dtok, n_tokens, cols / 8);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  embedding_bwd_pos_kernel<<<grid_for((int64_t)seq * (cols / 8), 256), 256, 0, stream>>>(reinterpret_cast<const uint4*>(dout), dpos, n_tokens, seq, cols / 8);
  return cudaGetLastError();
}

}  // namespace msb
