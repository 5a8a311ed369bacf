// Persistent, warp-specialised tcgen05 GEMM for sm_100a with fused mesh collectives.
// See sm100_gemm.h for the interface and the role of each argument.
//
// CTA pairs (clusters of two, 256 threads per CTA, one CTA per SM, static round-robin schedule of
// 256x256 cluster tiles; each CTA holds 128 rows of A and 128 columns of B of the pair's tile):
//   warp 0      TMA producer (both CTAs): waits for the chunk / panel flags a tile depends on, then
//               fills a ring of kStages (A 128x64, B 128x64) bf16 tiles in 128-byte-swizzled smem;
//               the loads complete on the leader CTA's mbarrier
//   warp 1      MMA issuer (leader CTA): one elected thread issues tcgen05.mma.cta_group::2
//               (M=256, N=256, K=16) into one of two 256-column fp32 accumulators in TMEM
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (one TMEM lane quarter per warp), then
//               either bias / GeLU and a store to local memory, or the push of the bf16 partial tile
//               into the owner GPU's slot (staged in smem, written with coalesced 16-byte stores or
//               2-D TMA tensor stores) with one arrival count per slice and owner
//   warps 6..7  communication and reduction (kAuxWarps of them; warp 6 of CTA 0 also runs the
//               cross-GPU entry / exit barrier).  Gather side: the warps of all CTAs share the pieces
//               of the LOCAL shard; a piece is read once with coalesced 16-byte loads (several per
//               lane in flight) and written with 16-byte stores to every GPU of the group (posted
//               writes over NVLink), one flag per chunk on every destination.  Reduce side: after
//               the gather the same warps sum, slice by slice and as soon as a slice's arrival
//               counter is complete, the partial tiles that peers pushed into this GPU's slots, so
//               the sums of slice s run under the tensor-core work of slice s + 1.
//
// Every wait is bounded (ptx.cuh); on expiry the kernel records a code in `status`, leaves
// its loops, frees TMEM and returns.
#include "sm100_gemm.h"

#include <cuda_bf16.h>

#include "../common/ptx.cuh"

namespace msb {

namespace {

constexpr uint32_t kAStageBytes = kBM * kBK * 2;        // 16 KiB: this CTA's 128 rows of A
constexpr uint32_t kBStageBytes = (kBN / 2) * kBK * 2;  // 16 KiB: this CTA's 128 columns of B
constexpr uint32_t kSmemA = 0;
constexpr uint32_t kSmemB = kSmemA + kStages * kAStageBytes;
constexpr uint32_t kSmemEpi = kSmemB + kStages * kBStageBytes;
constexpr uint32_t kSmemBar = kSmemEpi + 4 * kEpiStageBytes;
constexpr uint32_t kSmemCnt = kSmemBar + 256;   // [4 epilogue warps][kMaxPeers] tile counts
constexpr uint32_t kSmemTotal = kSmemCnt + 4 * kMaxPeers * 4;
constexpr uint32_t kSmemAlloc = kSmemTotal + 1024;  // slack for manual 1024-byte alignment
constexpr uint32_t kTmemCols = 512;
constexpr int kEpiThreads = 128;

// ---- CTA pair (cluster of two) helpers ----
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

// m_blk counts 256-row cluster tiles; a CTA of rank r works on rows (2 * m_blk + r) * 128.
struct TileCoord {
  int m_blk, n_blk, slice;
};

__device__ __forceinline__ TileCoord tile_coord(int t, const GemmArgs& a) {
  const int tiles_s = a.slice_dim == 0 ? a.tiles_m : a.tiles_n;
  const int tiles_o = a.slice_dim == 0 ? a.tiles_n : a.tiles_m;
  const int S = a.n_slices;
  const int nb = tiles_s / S;
  const int per_slice = nb * tiles_o;
  const int s = t / per_slice;
  const int r = t - s * per_slice;
  const int g_span = a.group * tiles_o;
  const int g = r / g_span;
  const int rr = r - g * g_span;
  const int g0 = g * a.group;
  const int geff = min(a.group, nb - g0);
  const int o = rr / geff;
  const int w = rr - o * geff;
  int jj = g0 + w + a.rot;
  if (jj >= nb) jj -= nb;
  const int cg = jj / a.cyc;
  const int blk_s = (cg * S + s) * a.cyc + (jj - cg * a.cyc);
  TileCoord c;
  c.m_blk = a.slice_dim == 0 ? blk_s : o;
  c.n_blk = a.slice_dim == 0 ? o : blk_s;
  c.slice = s;
  return c;
}

__device__ __forceinline__ void report(const GemmArgs& a, uint32_t code, uint32_t d0, uint32_t d1) {
  if (atomicCAS(a.status, 0u, code) == 0u) {
    a.status[1] = blockIdx.x;
    a.status[2] = d0;
    a.status[3] = d1;
  }
}

// Timeline of one launch (kernel instantiated with kTrace only): events are 16-byte records
// {globaltimer low, high, kind, argument} in a per-CTA area of a.trace whose first record is the event count.
// The untraced instantiation contains none of this.
template <bool kTrace>
__device__ __forceinline__ void trace_event(const GemmArgs& a, uint32_t kind, uint32_t arg) {
  if constexpr (kTrace) {
    uint4* area = reinterpret_cast<uint4*>(a.trace) + (size_t)blockIdx.x * (size_t)(a.trace_cap + 1);
    const uint32_t i = atomicAdd(reinterpret_cast<uint32_t*>(area), 1u);
    if (i < (uint32_t)a.trace_cap) {
      const uint64_t t = globaltimer_ns();
      area[1 + i] = make_uint4((uint32_t)t, (uint32_t)(t >> 32), kind, arg);
    }
  }
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// Waits for one chunk flag of an operand (bumped by this GPU's and by peers' communication warps).
// The value that means "complete" belongs to the operand (a_flag_target / b_flag_target), not to the
// chunk's position in the travel order: the chunk list is ordered by need, the flags by operand.
__device__ __forceinline__ bool wait_chunk(const GemmArgs& a, int idx, uint32_t target, uint64_t tmo) {
  return wait_flag_geq_sys(a.chunk_flags + idx, target, tmo);
}
// `seen` remembers chunks already observed complete, so that only the first tile that needs a
// chunk pays for the system-scope flag reads.
__device__ __forceinline__ bool wait_operand(const GemmArgs& a, int mode, int base, int count, uint32_t target,
                                             int slice, int col_chunk, uint64_t tmo, uint64_t& seen) {
  if (mode == 0 || mode == 3) return true;   // mode 3 is waited for inside the contraction loop
  const int lo = mode == 1 ? base + slice : (mode == 4 ? base + col_chunk : base);
  const int hi = (mode == 1 || mode == 4) ? lo + 1 : base + count;
  for (int i = lo; i < hi; ++i) {
    const uint64_t bit = 1ull << (i & 63);
    if (i < 64 && (seen & bit)) continue;
    if (!wait_chunk(a, i, target, tmo)) return false;
    if (i < 64) seen |= bit;
  }
  return true;
}

// K-panel schedule: flag `idx` counts to kp_target (one source GPU per panel).
__device__ __forceinline__ bool wait_panel(const GemmArgs& a, int idx, uint64_t tmo, uint64_t& seen,
                                           bool& fresh) {
  const uint64_t bit = 1ull << (idx & 63);
  if (idx < 64 && (seen & bit)) return true;
  if (!wait_flag_geq_sys(a.chunk_flags + idx, a.kp_target, tmo)) return false;
  if (idx < 64) seen |= bit;
  fresh = true;
  return true;
}

// ------------------------------------------------------------------------------------------
// communication / reduce warps
// ------------------------------------------------------------------------------------------
constexpr uint32_t kPieceBytes = 16384;   // work unit of the gather: one warp copies one piece
constexpr int kGatherUnroll = 8;          // 16-byte loads in flight per lane

__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_v4(void* p, const uint4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void aux_bar_sync() {   // the kAuxWarps warps of this CTA (named barrier 1)
  asm volatile("bar.sync 1, %0;" ::"n"(32 * kAuxWarps) : "memory");
}

// Copies `nvec` 16-byte vectors of a 2-D block (vpr vectors per row) from the local shard to every
// destination; vector v of the piece is element (v / vpr, v % vpr) counted from the piece's origin.
__device__ __forceinline__ void gather_piece(const char* src, uint64_t sp, uint64_t dp, uint32_t vpr,
                                             uint32_t nvec, const PushJob& job, uint64_t dst_off, int lane) {
  for (uint32_t v0 = 0; v0 < nvec; v0 += 32 * kGatherUnroll) {
    uint4 val[kGatherUnroll];
    uint64_t doff[kGatherUnroll];
#pragma unroll
    for (int u = 0; u < kGatherUnroll; ++u) {
      const uint32_t v = v0 + u * 32 + lane;
      if (v < nvec) {
        const uint32_t r = v / vpr, c = v - r * vpr;
        val[u] = ld_nc_v4(src + (uint64_t)r * sp + ((uint64_t)c << 4));
        doff[u] = dst_off + (uint64_t)r * dp + ((uint64_t)c << 4);
      }
    }
    for (uint32_t d = 0; d < job.n_dst; ++d) {
      char* dst = job.dst[d];
#pragma unroll
      for (int u = 0; u < kGatherUnroll; ++u)
        if (v0 + u * 32 + lane < nvec) st_v4(dst + doff[u], val[u]);
    }
  }
}

// Sums ROWS consecutive rows (8 columns per lane) over the first `n` of SLOTS slots in fixed
// order and writes them: ROWS x SLOTS 16-byte loads are in flight per lane.
template <int ROWS, int SLOTS>
__device__ __forceinline__ void reduce_rows(const GemmArgs& a, const __nv_bfloat16* slots, int64_t slot_stride,
                                            int n, int64_t row0, int col, const float (&bv)[8]) {
  uint4 x[ROWS][SLOTS];
#pragma unroll
  for (int rr = 0; rr < ROWS; ++rr) {
#pragma unroll
    for (int sl = 0; sl < SLOTS; ++sl)
      if (sl < n && row0 + rr < a.red_rows)
        x[rr][sl] = *reinterpret_cast<const uint4*>(slots + sl * slot_stride + (row0 + rr) * a.red_ld + col);
  }
#pragma unroll
  for (int rr = 0; rr < ROWS; ++rr) {
    const int64_t row = row0 + rr;
    if (row >= a.red_rows) continue;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
    for (int sl = 0; sl < SLOTS; ++sl)
      if (sl < n) {
        const uint4 v = x[rr][sl];
        acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x);
        acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
        acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z);
        acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
      }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += bv[i];
    if (a.c_fp32) {
      float* p = reinterpret_cast<float*>(a.C) + row * a.ldc + col;
      float4 lo = make_float4(acc[0], acc[1], acc[2], acc[3]);
      float4 hi = make_float4(acc[4], acc[5], acc[6], acc[7]);
      if (a.accumulate) {
        const float4 c0 = *reinterpret_cast<const float4*>(p);
        const float4 c1 = *reinterpret_cast<const float4*>(p + 4);
        lo.x += c0.x; lo.y += c0.y; lo.z += c0.z; lo.w += c0.w;
        hi.x += c1.x; hi.y += c1.y; hi.z += c1.z; hi.w += c1.w;
      }
      *reinterpret_cast<float4*>(p) = lo;
      *reinterpret_cast<float4*>(p + 4) = hi;
    } else {
      __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(a.C) + row * a.ldc + col;
      if (a.accumulate) {
        const uint4 c = *reinterpret_cast<const uint4*>(p);
        acc[0] += bf16_lo(c.x); acc[1] += bf16_hi(c.x);
        acc[2] += bf16_lo(c.y); acc[3] += bf16_hi(c.y);
        acc[4] += bf16_lo(c.z); acc[5] += bf16_hi(c.z);
        acc[6] += bf16_lo(c.w); acc[7] += bf16_hi(c.w);
      }
      uint4 o4;
      o4.x = pack_bf16(acc[0], acc[1]);
      o4.y = pack_bf16(acc[2], acc[3]);
      o4.z = pack_bf16(acc[4], acc[5]);
      o4.w = pack_bf16(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(p) = o4;
    }
  }
}

// Sums the partial tiles of slice `s` that the push group's ranks wrote into this GPU's slots.
// Work unit: 32 rows x 256 columns of one block.  Warps take units from a per-slice counter, so the
// communication warps start a slice while the tiles of the next one run and the epilogue warps of a
// CTA that has finished its tiles help with what is left.  Every unit is summed by one warp in fixed
// order (slot 0, 1, ...): the result does not depend on arrival order nor on who took the unit.
__device__ __noinline__ void reduce_slice(const GemmArgs& a, int s, int lane) {
  const int RB = a.red_slice_dim == 0 ? 2 * kBM : kBM;
  const int tiles_r = (a.red_rows + RB - 1) / RB;
  const int tiles_c = (a.red_cols + kBN - 1) / kBN;
  const int tiles_s = a.red_slice_dim == 0 ? tiles_r : tiles_c;
  const int tiles_o = a.red_slice_dim == 0 ? tiles_c : tiles_r;
  const int S = a.n_slices;
  const int nb = tiles_s / S;
  const int sub = RB / 32;                       // units per block
  const int n_units = nb * tiles_o * sub;
  const __nv_bfloat16* slots = reinterpret_cast<const __nv_bfloat16*>(a.red_slots);
  const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(a.bias);
  const int64_t slot_stride = (int64_t)a.red_rows * a.red_ld;
  for (;;) {
    int u = 0;
    if (lane == 0) u = (int)atomicAdd(a.red_work + s, 1u);
    u = __shfl_sync(0xffffffffu, u, 0);
    if (u >= n_units) break;
    const int blk = u / sub, part = u - blk * sub;
    const int j = blk / tiles_o, o = blk - j * tiles_o;
    const int cg = j / a.cyc;
    const int blk_s = (cg * S + s) * a.cyc + (j - cg * a.cyc);
    const int rb = a.red_slice_dim == 0 ? blk_s : o;
    const int cb = a.red_slice_dim == 0 ? o : blk_s;
    const int col = cb * kBN + lane * 8;
    if (col >= a.red_cols) continue;
    float bv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (bias != nullptr) {
#pragma unroll
      for (int i = 0; i < 8; ++i) bv[i] = __bfloat162float(bias[col + i]);
    }
    const int64_t row0 = (int64_t)rb * RB + part * 32;
    if (a.red_n <= 2) {
#pragma unroll 1
      for (int r = 0; r < 32; r += 8) reduce_rows<8, 2>(a, slots, slot_stride, a.red_n, row0 + r, col, bv);
    } else if (a.red_n <= 4) {
#pragma unroll 1
      for (int r = 0; r < 32; r += 4) reduce_rows<4, 4>(a, slots, slot_stride, a.red_n, row0 + r, col, bv);
    } else {
#pragma unroll 1
      for (int r = 0; r < 32; r += 2) reduce_rows<2, 8>(a, slots, slot_stride, a.red_n, row0 + r, col, bv);
    }
  }
}

template <bool kTrace>
__device__ void aux_warp_main(const GemmArgs& a, int aux) {
  const int lane = threadIdx.x & 31;
  const uint64_t tmo = a.timeout_ns;
  const int worker = blockIdx.x * kAuxWarps + aux;
  const int n_workers = gridDim.x * kAuxWarps;
  bool ok = true;

  // ---- entry barrier: warp 6 of CTA 0 tells every rank that this GPU's earlier work is complete
  //      and waits for the same message from every rank, then releases the local CTAs.
  if (a.n_ranks > 0) {
    if (blockIdx.x == 0 && aux == 0) {
      if (lane < a.n_ranks && lane != a.my_rank) {
        st_release_sys(a.entry_flags[lane] + a.my_rank, a.epoch);
        if (!wait_flag_geq_sys(a.entry_flags[a.my_rank] + lane, a.epoch, tmo)) {
          report(a, kTimeoutEntry, lane, a.epoch);
          ok = false;
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (lane == 0 && ok) st_release_gpu(a.go_flag, a.epoch);
    } else {
      if (lane == 0) {
        if (!wait_flag_geq_gpu(a.go_flag, a.epoch, 2 * tmo)) {
          report(a, kTimeoutGo, 0, a.epoch);
          ok = false;
        }
      }
      ok = __all_sync(0xffffffffu, ok);
    }
  }

  // ---- gather side: the pieces of every chunk are dealt round-robin to the aux warps of all CTAs
  if (ok && a.n_chunks > 0 && !a.skip_comm) {
    uint32_t running = 0;   // pieces of earlier jobs (keeps the round-robin going across jobs)
    for (int c = 0; c < a.n_chunks; ++c) {
      const ChunkDesc& cd = a.chunks[c];
      for (int jn = cd.job_begin; jn < cd.job_end; ++jn) {
        const PushJob& j = a.jobs[jn];
        const char* base = a.gather_src[j.src_sel & 1] + j.src_off;
        const uint32_t vpr = j.row_bytes >> 4;
        uint32_t segs = 1, rows_pp, pieces;
        if (j.row_bytes > kPieceBytes) {          // long rows: segments of one row
          segs = (j.row_bytes + kPieceBytes - 1) / kPieceBytes;
          rows_pp = 1;
          pieces = j.rows * segs;
        } else {
          rows_pp = kPieceBytes / j.row_bytes;
          pieces = (j.rows + rows_pp - 1) / rows_pp;
        }
        uint32_t first = ((uint32_t)worker + (uint32_t)n_workers - running % (uint32_t)n_workers) % (uint32_t)n_workers;
        for (uint32_t pi = first; pi < pieces; pi += n_workers) {
          if (segs > 1) {
            const uint32_t row = pi / segs, seg = pi - row * segs;
            const uint32_t off = seg * kPieceBytes;
            const uint32_t bytes = min(kPieceBytes, j.row_bytes - off);
            gather_piece(base + (uint64_t)row * j.src_pitch + off, j.src_pitch, j.dst_pitch, bytes >> 4,
                         bytes >> 4, j, (uint64_t)row * j.dst_pitch + off, lane);
          } else {
            const uint32_t row0 = pi * rows_pp;
            const uint32_t rows = min(rows_pp, j.rows - row0);
            gather_piece(base + (uint64_t)row0 * j.src_pitch, j.src_pitch, j.dst_pitch, vpr, rows * vpr, j,
                         (uint64_t)row0 * j.dst_pitch, lane);
          }
        }
        running += pieces;
      }
      // this warp's share of the chunk has been written everywhere: tell every destination
      __threadfence_system();
      __syncwarp();
      if (lane < (int)cd.n_sig) red_add_release_sys(cd.sig[lane], 1u);
      __syncwarp();
      if (lane == 0) trace_event<kTrace>(a, kTraceChunkSent, (uint32_t)c);
    }
  }

  // ---- optional exit barrier: nobody leaves before every rank has finished its transfers
  if (a.n_ranks > 0 && a.exit_barrier) {
    aux_bar_sync();   // all aux warps of this CTA are done with the gather
    if (aux == 0) {
      if (lane == 0) red_add_release_gpu(a.done_counter, 1u);
      if (blockIdx.x == 0) {
        bool ok2 = ok;
        if (lane == 0 && ok2) {
          if (!wait_flag_geq_gpu(a.done_counter, a.done_target, 6 * tmo)) {
            report(a, kTimeoutExit, 0xffffffffu, a.epoch);
            ok2 = false;
          }
        }
        ok2 = __all_sync(0xffffffffu, ok2);
        if (ok2 && lane < a.n_ranks && lane != a.my_rank) {
          st_release_sys(a.exit_flags[lane] + a.my_rank, a.epoch);
          if (!wait_flag_geq_sys(a.exit_flags[a.my_rank] + lane, a.epoch, 6 * tmo))
            report(a, kTimeoutExit, lane, a.epoch);
        }
      }
    }
  }

  // ---- reduce side: slice by slice, as soon as every partial tile of the slice has arrived
  if (a.red_n > 0) {
    for (int s = 0; s < a.n_slices && ok; ++s) {
      if (lane == 0) {
        if (!wait_flag_geq_sys(a.red_counter + s, a.red_target, 8 * tmo)) {
          report(a, kTimeoutReduce, s, worker);
          ok = false;
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        if (lane == 0) trace_event<kTrace>(a, kTraceSumBegin, (uint32_t)s);
        reduce_slice(a, s, lane);
        if (lane == 0) trace_event<kTrace>(a, kTraceSumEnd, (uint32_t)s);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// epilogue helpers
// ------------------------------------------------------------------------------------------
// Stores 32 consecutive columns of one row.  `v` holds fp32 accumulators.
__device__ __forceinline__ void store_row32(const GemmArgs& a, void* base, int64_t ld, bool fp32,
                                            bool accumulate, int64_t row, int col0, int ncols_valid,
                                            float (&v)[32]) {
  if (fp32) {
    float* p = reinterpret_cast<float*>(base) + row * ld + col0;
    if (ncols_valid == 32) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        if (accumulate) {
          float4 c = *reinterpret_cast<const float4*>(p + i);
          o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
        }
        *reinterpret_cast<float4*>(p + i) = o;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncols_valid) p[i] = accumulate ? p[i] + v[i] : v[i];
    }
  } else {
    __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(base) + row * ld + col0;
    if (ncols_valid == 32) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 o;
        if (accumulate) {
          uint4 c = *reinterpret_cast<const uint4*>(p + i);
          o.x = pack_bf16(v[i] + bf16_lo(c.x), v[i + 1] + bf16_hi(c.x));
          o.y = pack_bf16(v[i + 2] + bf16_lo(c.y), v[i + 3] + bf16_hi(c.y));
          o.z = pack_bf16(v[i + 4] + bf16_lo(c.z), v[i + 5] + bf16_hi(c.z));
          o.w = pack_bf16(v[i + 6] + bf16_lo(c.w), v[i + 7] + bf16_hi(c.w));
        } else {
          o.x = pack_bf16(v[i], v[i + 1]);
          o.y = pack_bf16(v[i + 2], v[i + 3]);
          o.z = pack_bf16(v[i + 4], v[i + 5]);
          o.w = pack_bf16(v[i + 6], v[i + 7]);
        }
        *reinterpret_cast<uint4*>(p + i) = o;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (i >= ncols_valid) continue;
        float x = v[i];
        if (accumulate) x += __bfloat162float(p[i]);
        p[i] = __float2bfloat16_rn(x);
      }
    }
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------
// kernel
// ------------------------------------------------------------------------------------------
template <bool kTrace>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
sm100_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                  const __grid_constant__ PushMaps pmaps, const __grid_constant__ GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem + kSmemA;
  uint8_t* sB = smem + kSmemB;
  uint8_t* sEpi = smem + kSmemEpi;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemBar);
  uint32_t* sCnt = reinterpret_cast<uint32_t*>(smem + kSmemCnt);
  uint64_t* full_bar = bars;                   // [kStages]
  uint64_t* empty_bar = bars + kStages;        // [kStages]
  uint64_t* tfull_bar = bars + 2 * kStages;    // [2]
  uint64_t* tempty_bar = tfull_bar + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0: leader of the CTA pair (issues the MMAs)
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const uint64_t tmo = a.timeout_ns;
  const int num_tiles = a.tiles_m * a.tiles_n;   // 256 x 256 cluster tiles
  // Deep push staging gives up the last pipeline stage: its A and B buffers become the second and
  // third staging buffer of each epilogue warp (more tensor stores in flight towards the owners).
  const bool deep_push = a.push_n > 0 && a.push_bufs >= 3 && a.push_mode == 0;
  const uint32_t nst = deep_push ? kStages - 1 : kStages;
  const int kblocks = (a.K + kBK - 1) / kBK;

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(full_bar + i, 1);    // used in the leader: both CTAs' loads complete on it
      mbar_init(empty_bar + i, 1);   // one per CTA
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull_bar + i, 1);                  // one per CTA
      mbar_init(tempty_bar + i, 2 * kEpiThreads);   // used in the leader: both CTAs' epilogues
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before_sync();
  cluster_sync_all();   // both CTAs' barriers exist before any remote arrival or commit
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      bool ok = true;
      if (a.n_ranks > 0 && num_tiles > 0) {
        if (!wait_flag_geq_gpu(a.go_flag, a.epoch, 2 * tmo)) {
          report(a, kTimeoutGo, 1, a.epoch);
          ok = false;
        }
      }
      uint32_t stage = 0, phase = 0;
      uint64_t seen = 0;
      const bool kpanels = a.a_flag_mode == 3 || a.b_flag_mode == 3;
      for (int t = cluster_id; t < num_tiles && ok; t += n_clusters) {
        const TileCoord tc = tile_coord(t, a);
        if (a.a_flag_mode | a.b_flag_mode) {
          const uint64_t before = seen;
          const int cc = tc.n_blk / a.b_nchunk;   // column chunk of B (flag mode 4)
          if (!wait_operand(a, a.a_flag_mode, a.a_flag_base, a.a_flag_count, a.a_flag_target, tc.slice, 0,
                            3 * tmo, seen) ||
              !wait_operand(a, a.b_flag_mode, a.b_flag_base, a.b_flag_count, a.b_flag_target, tc.slice, cc,
                            3 * tmo, seen)) {
            report(a, kTimeoutChunk, t, tc.slice);
            ok = false;
            break;
          }
          if (seen != before || a.n_chunks > 64) fence_proxy_async();
          trace_event<kTrace>(a, kTraceOperandsReady, (uint32_t)t);
        }
        const int row_a = (2 * tc.m_blk + (int)rank) * kBM;        // this CTA's 128 rows of A
        const int col_b = tc.n_blk * kBN + (int)rank * (kBN / 2);  // this CTA's 128 columns of B
        for (int kb0 = 0; kb0 < kblocks; ++kb0) {
          int kb = kb0 + a.k_rot;   // the contraction loop may start anywhere: sums commute
          if (kb >= kblocks) kb -= kblocks;
          if (kpanels) {
            // K-panel schedule: the first k-block of a panel waits for the panel's flag
            bool fresh = false;
            if (a.a_flag_mode == 3 && (kb0 == 0 || kb % a.a_kpanel == 0))
              ok = ok && wait_panel(a, a.a_flag_base + kb / a.a_kpanel, 3 * tmo, seen, fresh);
            if (a.b_flag_mode == 3 && (kb0 == 0 || kb % a.b_kpanel == 0))
              ok = ok && wait_panel(a, a.b_flag_base + kb / a.b_kpanel, 3 * tmo, seen, fresh);
            if (!ok) {
              report(a, kTimeoutChunk, t, 0x10000u + kb);
              break;
            }
            if (fresh) fence_proxy_async();
          }
          if (!mbar_wait(empty_bar + stage, phase ^ 1, 5 * tmo)) {
            report(a, kTimeoutEmpty, t, kb);
            ok = false;
            break;
          }
          const uint32_t fb = mapa_u32(smem_u32(full_bar + stage), 0);   // the leader's barrier
          if (rank == 0) mbar_expect_tx(full_bar + stage, 2 * (kAStageBytes + kBStageBytes));
          uint8_t* da = sA + stage * kAStageBytes;
          uint8_t* db = sB + stage * kBStageBytes;
          // an MN-major operand is one 3-D box per stage (two 64-wide blocks of 64 k-rows) when its
          // extent allows it, else two 2-D boxes: the producer's issue rate is what bounds the pipe
          if (!a.a_mn_major) {
            tma_load_2d_pair(da, &tma_a, fb, kb * kBK, row_a);
          } else if (a.a_map3d) {
            tma_load_3d_pair(da, &tma_a, fb, 0, kb * kBK, row_a >> 6);
          } else {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)
              tma_load_2d_pair(da + j * (kBK * 128), &tma_a, fb, row_a + j * 64, kb * kBK);
          }
          if (!a.b_mn_major) {
            tma_load_2d_pair(db, &tma_b, fb, kb * kBK, col_b);
          } else if (a.b_map3d) {
            tma_load_3d_pair(db, &tma_b, fb, 0, kb * kBK, col_b >> 6);
          } else {
#pragma unroll
            for (int j = 0; j < kBN / 128; ++j)
              tma_load_2d_pair(db + j * (kBK * 128), &tma_b, fb, col_b + j * 64, kb * kBK);
          }
          if (++stage == nst) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc_bf16(2 * kBM, kBN, a.a_mn_major, a.b_mn_major);
      const uint32_t a_lbo = a.a_mn_major ? kBK * 128 : 16;
      const uint32_t b_lbo = a.b_mn_major ? kBK * 128 : 16;
      const uint32_t a_kstep = a.a_mn_major ? 16 * 128 : 32;  // bytes per K=16 step
      const uint32_t b_kstep = a.b_mn_major ? 16 * 128 : 32;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = cluster_id; t < num_tiles && ok; t += n_clusters, ++it) {
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar + acc, acc_phase ^ 1, 6 * tmo)) {
          report(a, kTimeoutTmemEmpty, t, acc);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * kBN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar + stage, phase, 4 * tmo)) {
            report(a, kTimeoutFull, t, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(sA + stage * kAStageBytes);
          const uint32_t sb = smem_u32(sB + stage * kBStageBytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = make_smem_desc(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t db = make_smem_desc(sb + k * b_kstep, b_lbo, 1024);
            umma_f16_pair(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          const uint32_t eb = smem_u32(empty_bar + stage);
          umma_commit_pair(eb);                // this CTA's stage is free again
          umma_commit_pair(mapa_u32(eb, 1));   // and so is the peer's
          if (++stage == nst) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          const uint32_t tb = smem_u32(tfull_bar + acc);
          umma_commit_pair(tb);
          umma_commit_pair(mapa_u32(tb, 1));
        }
      }
    }
  } else if (warp < 6) {
    // ===================== epilogue =====================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(a.bias);
    bool ok = true;
    int it = 0;
    int push_seq = 0;          // staging buffer of the next band (deep push: three per warp)
    // Push path: arrivals are counted at the owners once per slice, not per tile.  Ordering a tile's
    // stores before its counter costs an NVLink round trip (system-scope fence), so this warp sums
    // its tiles per owner in shared memory and pays that round trip when the slice changes.
    uint32_t* cnt = sCnt + (warp - 2) * kMaxPeers;
    int cur_slice = -1;
    if (lane < kMaxPeers) cnt[lane] = 0;
    __syncwarp();
    auto flush_counts = [&](int slice) {
      if (a.push_mode == 0 && lane == 0) {
        bulk_wait_all<0>();     // this warp's tensor stores have completed
        fence_proxy_async();
      }
      __threadfence_system();
      __syncwarp();
      if (lane < a.push_n) {
        const uint32_t c = cnt[lane];
        if (c != 0) {
          red_add_release_sys(a.push_counter[lane] + slice, c);
          cnt[lane] = 0;
        }
      }
      __syncwarp();
    };
    for (int t = cluster_id; t < num_tiles && ok; t += n_clusters, ++it) {
      const TileCoord tc = tile_coord(t, a);
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
      const int m_blk = 2 * tc.m_blk + (int)rank;   // this CTA's 128-row block
      const uint32_t te_leader = mapa_u32(smem_u32(tempty_bar + acc), 0);
      // lane 0 does the bounded wait and the warp follows its verdict, so the warp-wide
      // tcgen05.ld below is never reached by only some of the lanes
      int okw = 1;
      if (lane == 0) okw = mbar_wait(tfull_bar + acc, acc_phase, 7 * tmo) ? 1 : 0;
      okw = __shfl_sync(0xffffffffu, okw, 0);
      if (!okw) {
        if (lane == 0) report(a, kTimeoutTmemFull, t, acc);
        ok = false;
        break;
      }
      mbar_wait(tfull_bar + acc, acc_phase, tmo);  // already complete: orders this lane's reads
      tc_fence_after_sync();
      if (warp == 2 && lane == 0) trace_event<kTrace>(a, kTraceTileComputed, (uint32_t)t);
      if (a.push_n > 0 && tc.slice != cur_slice) {
        if (cur_slice >= 0) flush_counts(cur_slice);
        cur_slice = tc.slice;
      }
      const int64_t row = (int64_t)m_blk * kBM + q * 32 + lane;
      const bool row_ok = row < a.M;
      // destination of this tile
      void* out = a.C;
      int64_t ld = a.ldc;
      bool out_fp32 = a.c_fp32 != 0, accum = a.accumulate != 0;
      int64_t orow = row;
      int ocol_shift = 0;
      int owner = 0;
      if (a.push_n > 0) {
        const int c0 = a.push_dim == 0 ? m_blk * kBM : tc.n_blk * kBN;
        owner = c0 / a.push_extent;
        out = a.push_base[owner];
        ld = a.push_ld;
        out_fp32 = false;
        accum = false;
        if (a.push_dim == 0) orow = row - (int64_t)owner * a.push_extent;
        else ocol_shift = owner * a.push_extent;
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kBN;
      if (a.push_n > 0) {
        // Push path: 64 columns at a time go through this warp's 4 KiB staging buffer (128-byte
        // swizzled, so the lanes' row writes spread over the banks) and leave for the owner's slot
        // either as coalesced 16-byte stores read back row-major (push_mode 1) or as ONE 2-D TMA
        // tensor store of 32 rows x 128 bytes (push_mode 0); both are posted writes over NVLink.
        uint8_t* stage_buf[3];
        stage_buf[0] = sEpi + (warp - 2) * kEpiStageBytes;
        stage_buf[1] = sA + (kStages - 1) * kAStageBytes + (warp - 2) * kEpiStageBytes;
        stage_buf[2] = sB + (kStages - 1) * kBStageBytes + (warp - 2) * kEpiStageBytes;
        const CUtensorMap* omap = &pmaps.m[owner];
        const int32_t y0 = (int32_t)(orow - lane);   // first row of this warp's 32-row band
#pragma unroll 1
        for (int c2 = 0; c2 < kBN / 64; ++c2) {
          uint32_t r0[32], r1[32];
          __syncwarp();
          tmem_ld_32x32(taddr + c2 * 64, r0);
          tmem_ld_32x32(taddr + c2 * 64 + 32, r1);
          tmem_ld_wait();
          if (c2 == kBN / 64 - 1) {
            tc_fence_before_sync();
            mbar_arrive_cluster(te_leader);
          }
          // the store that last used this staging buffer has left it
          uint8_t* stage = stage_buf[0];
          if (deep_push) {
            stage = push_seq == 0 ? stage_buf[0] : (push_seq == 1 ? stage_buf[1] : stage_buf[2]);
            if (++push_seq == 3) push_seq = 0;
            if (lane == 0) bulk_wait_read<2>();
          } else if (a.push_mode == 0) {
            if (lane == 0) bulk_wait_read<0>();
          }
          __syncwarp();
          uint8_t* srow = stage + lane * 128;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t* r = k < 4 ? r0 : r1;
            const int b = (k & 3) * 8;
            uint4 u;
            u.x = pack_bf16(__uint_as_float(r[b + 0]), __uint_as_float(r[b + 1]));
            u.y = pack_bf16(__uint_as_float(r[b + 2]), __uint_as_float(r[b + 3]));
            u.z = pack_bf16(__uint_as_float(r[b + 4]), __uint_as_float(r[b + 5]));
            u.w = pack_bf16(__uint_as_float(r[b + 6]), __uint_as_float(r[b + 7]));
            *reinterpret_cast<uint4*>(srow + ((k ^ (lane & 7)) << 4)) = u;
          }
          if (a.push_mode == 1) {
            // Read the band back row-major (4 rows x 128 bytes per instruction, conflict-free through
            // the same swizzle) and write it with ordinary 16-byte stores: posted writes that the
            // load/store units keep in flight by the hundred, unlike the bulk-store engine.
            __syncwarp();
            char* gband = reinterpret_cast<char*>(out) +
                          (((orow - lane) * ld) + (tc.n_blk * kBN + c2 * 64 - ocol_shift)) * 2;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = i * 4 + (lane >> 3), ch = lane & 7;
              const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((ch ^ (rr & 7)) << 4));
              *reinterpret_cast<uint4*>(gband + (int64_t)rr * ld * 2 + ch * 16) = v;
            }
            continue;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int32_t x0 = tc.n_blk * kBN + c2 * 64 - ocol_shift;
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(omap), "r"(smem_u32(stage)), "r"(x0), "r"(y0)
                         : "memory");
            bulk_commit();
          }
        }
        if (lane == 0) cnt[owner] += 1;
        if (warp == 2 && lane == 0) trace_event<kTrace>(a, kTraceTilePushed, (uint32_t)t);
      } else {
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
          uint32_t r[32];
          __syncwarp();
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (c == kBN / 32 - 1) {
            // accumulator fully read: hand it back to the leader's MMA warp
            tc_fence_before_sync();
            mbar_arrive_cluster(te_leader);
          }
          const int col0 = tc.n_blk * kBN + c * 32;
          const int nvalid = min(32, a.N - col0);
          if (row_ok && nvalid > 0) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            if (bias != nullptr) {
              for (int i = 0; i < 32; ++i)
                if (i < nvalid) v[i] += __bfloat162float(bias[col0 + i]);
            }
            if (a.act == 1) {
              if (a.C_pre != nullptr)
                store_row32(a, a.C_pre, ld, false, false, orow, col0, nvalid, v);
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
            }
            store_row32(a, out, ld, out_fp32, accum, orow, col0, nvalid, v);
          }
        }
      }
    }
    if (cur_slice >= 0) flush_counts(cur_slice);
    // this CTA's tiles are done: help the communication warps with the slot sums that are left
    if (a.red_n > 0) {
      for (int s = 0; s < a.n_slices && ok; ++s) {
        int okw = 1;
        if (lane == 0 && !wait_flag_geq_sys(a.red_counter + s, a.red_target, 8 * tmo)) {
          report(a, kTimeoutReduce, s, 0x1000u + warp);
          okw = 0;
        }
        ok = __all_sync(0xffffffffu, okw) != 0;
        if (ok) reduce_slice(a, s, lane);
      }
    }
  } else {
    // ===================== communication / reduce warps =====================
    aux_warp_main<kTrace>(a, warp - 6);
  }

  // ---- all roles of both CTAs of the pair are done with TMEM, barriers and the pipeline
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");

}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
size_t sm100_gemm_smem_bytes() { return kSmemAlloc; }

cudaError_t launch_sm100_gemm(const CUtensorMap& tma_a, const CUtensorMap& tma_b,
                              const PushMaps& push_maps, const GemmArgs& args, int grid,
                              cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(sm100_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kSmemAlloc);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(sm100_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kSmemAlloc);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  if (args.trace != nullptr) {
    if (args.trace_cap <= 0 || (reinterpret_cast<uintptr_t>(args.trace) & 15)) return cudaErrorInvalidValue;
    sm100_gemm_kernel<true><<<grid, kGemmThreads, kSmemAlloc, stream>>>(tma_a, tma_b, push_maps, args);
  } else {
    sm100_gemm_kernel<false><<<grid, kGemmThreads, kSmemAlloc, stream>>>(tma_a, tma_b, push_maps, args);
  }
  return cudaGetLastError();
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer) {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || p == nullptr) return -1;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int make_tensor_map_mn3d(CUtensorMap* map, const void* base, uint64_t mn_extent, uint64_t k_rows,
                         uint64_t pitch_bytes, uint32_t blocks_per_box) {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || p == nullptr) return -1;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  if (mn_extent % 64 != 0) return -2;
  cuuint64_t dims[3] = {64, k_rows, mn_extent / 64};
  cuuint64_t strides[2] = {pitch_bytes, 128};
  cuuint32_t box[3] = {64, (cuuint32_t)kBK, blocks_per_box};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace msb
