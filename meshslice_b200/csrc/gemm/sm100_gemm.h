// Host-visible interface of the persistent tcgen05 GEMM with fused mesh collectives.
//
// One kernel computes  C[M,N] = op(A) * op(B)  (bf16 inputs, fp32 accumulation in TMEM) and,
// when asked to, also moves the data of the surrounding 2-D tensor-parallel collectives:
//   * gather side (all-gather -> GEMM): the communication warps of every CTA read pieces of this
//     GPU's shard and write them into the staging buffers of all GPUs of the group with 16-byte
//     peer stores over NVLink, then bump one flag per chunk on each of them; the TMA producer
//     warp waits for the flag of the chunk a tile needs.
//   * "push" side (GEMM -> reduce-scatter): the epilogue stores each partial tile straight
//     into the slot buffer of the GPU that owns it (peer stores over NVLink) and bumps a
//     per-slice counter there; the owner's communication warps (and epilogue warps that have
//     run out of tiles) sum the slots of a slice as soon as its counter is complete.
// This covers the three MeshSlice dataflows of the reference (TensorParallel.py:153-214):
// OS = gather A and B, LS = gather B and push over columns, RS = gather A and push over rows.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace msb {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;
#ifndef MSB_STAGES
#define MSB_STAGES 6
#endif
constexpr int kStages = MSB_STAGES;
constexpr int kMaxPeers = 8;
constexpr int kAuxWarps = 2;       // communication / reduce warps per CTA
constexpr int kGemmThreads = 32 * (6 + kAuxWarps);  // TMA, MMA, 4x epilogue, kAuxWarps x communication
constexpr int kEpiStageBytes = 32 * 128;  // per epilogue warp: 32 rows x 64 bf16 columns, 128-byte swizzled

// Error codes written to the status word (first error wins).
enum GemmStatus : uint32_t {
  kOk = 0,
  kTimeoutEmpty = 1,      // producer waited too long for a free pipeline stage
  kTimeoutFull = 2,       // MMA warp waited too long for TMA data
  kTimeoutTmemEmpty = 3,  // MMA warp waited too long for the epilogue to drain TMEM
  kTimeoutTmemFull = 4,   // epilogue waited too long for the accumulator
  kTimeoutChunk = 5,      // producer waited too long for a gathered chunk
  kTimeoutComm = 6,       // communication warp waited too long for a bulk copy
  kTimeoutEntry = 7,      // entry barrier with peers timed out
  kTimeoutExit = 8,       // exit barrier with peers timed out
  kTimeoutReduce = 9,     // reduce phase waited too long for peers' partial tiles
  kTimeoutGo = 10,        // CTA waited too long for the local "peers are ready" flag
};

// One 2-D copy of the gather side: a block of THIS GPU's shard is read once and written into
// the staging buffer of every GPU of the gathering group (own GPU included) with posted bulk
// stores over NVLink.  All addresses 16-byte aligned, row_bytes % 16 == 0.
struct PushJob {
  uint64_t src_off;       // byte offset inside the local source tensor gather_src[src_sel]
  uint32_t rows;
  uint32_t row_bytes;
  uint64_t src_pitch;
  uint64_t dst_pitch;
  uint32_t n_dst;
  uint32_t src_sel;       // which of GemmArgs::gather_src holds the block
  char* dst[kMaxPeers];   // same block inside each destination GPU's staging buffer
};

// One chunk of the gather: its jobs, the flag word to bump on every destination GPU once this
// CTA's share of the chunk has landed there, and the flag value that means "complete" on the
// consumer (CTAs per GPU x GPUs contributing to the chunk).
struct ChunkDesc {
  int job_begin, job_end;
  uint32_t n_sig;
  uint32_t target;
  uint32_t* sig[kMaxPeers];
};

// One 2-D copy by pulling (stand-alone P2P collectives): src may be peer memory.
struct CopyJob {
  const char* src;
  char* dst;
  uint32_t rows;
  uint32_t row_bytes;
  uint64_t src_pitch;
  uint64_t dst_pitch;
};

// Tensor maps of the owners' slot buffers for the push side ({64, 32} boxes, 128-byte swizzle).
struct PushMaps {
  CUtensorMap m[kMaxPeers];
};

struct GemmArgs {
  // ---- problem ----
  int M, N, K;
  int a_mn_major;  // 0: A stored [M,K] row-major; 1: A stored [K,M] row-major
  int b_mn_major;  // 0: B stored [N,K] row-major; 1: B stored [K,N] row-major
  int a_map3d;     // the tensor map of an MN-major A / B is the 3-D form of make_tensor_map_mn3d
  int b_map3d;
  // ---- local epilogue (used when push_n == 0) ----
  void* C;
  int64_t ldc;
  int c_fp32;          // 1: C is float, 0: C is bf16
  int accumulate;      // 1: C += result
  const void* bias;    // bf16 [N] or null
  int act;             // 0: none, 1: tanh-GeLU
  void* C_pre;         // bf16, same layout as C: pre-activation copy (act != 0), may be null
  // ---- tile order ----
  int tiles_m, tiles_n;  // tiles_m counts 256-row cluster tiles (two CTAs x 128 rows)
  int slice_dim;       // 0: slices over M blocks, 1: slices over N blocks
  int n_slices;        // block-cyclic slices of the sliced dimension (divides its tile count)
  int group;           // raster group size along the sliced dimension
  int cyc;             // tiles per cyclic block: slice s holds blocks (g*n_slices + s)*cyc + w
  int rot;             // rotation of the block order inside a slice (ranks of a push group start at
                       // different owners, so no owner's NVLink ingress is hit by all ranks at once)
  // ---- gather side (all-gather -> GEMM) ----
  const PushJob* jobs;
  const char* gather_src[2];   // local shards the jobs read from (so plans do not depend on them)
  const ChunkDesc* chunks;     // [n_chunks]
  int n_chunks;
  int skip_comm;               // 1: this launch moves no data (the chunks were filled earlier)
  uint32_t* chunk_flags;       // [n_chunks] local flags, bumped by every contributing CTA
  int a_flag_mode;             // 0: none, 1: flag a_flag_base + slice(tile), 2: all of [base, base+count),
                               // 3: K panels (below), 4 (B only): flag b_flag_base + n_block / b_nchunk
  int a_flag_base, a_flag_count;
  int b_flag_mode;
  int b_flag_base, b_flag_count;
  int b_nchunk;                // flag mode 4: 256-column blocks of B per chunk (>= 1)
  uint32_t a_flag_target;      // flag value once a chunk of A / of B is complete (modes 1, 2, 4):
  uint32_t b_flag_target;      // communication warps per GPU x GPUs contributing to the operand
  // flag mode 3 ("K panels", the SUMMA / ring schedules): the operand arrives in panels of the
  // contraction dimension; k-block kb needs flag base + kb / kpanel, which counts to kp_target
  int a_kpanel, b_kpanel;      // 64-wide k-blocks per panel
  uint32_t kp_target;
  int k_rot;                   // first k-block of every tile (the contraction loop wraps around), so
                               // that a rank can start with the panel it already holds
  // ---- push side ----
  int push_n;                  // number of owners (0: local epilogue)
  int push_dim;                // 0: owners split M, 1: owners split N
  int push_extent;             // rows (or columns) owned by each owner
  int push_mode;               // 0: 2-D TMA tensor stores, 1: ordinary 16-byte stores from the staging buffer
  int push_bufs;               // staging buffers per epilogue warp: 1, or 3 (then one pipeline stage fewer)
  void* push_base[kMaxPeers];  // owner o's slot for this source (bf16 [rows_local, ld])
  int64_t push_ld;
  uint32_t* push_counter[kMaxPeers];  // owner o's per-slice arrival counters
  // ---- reduce phase (runs on the owner after its tiles) ----
  int red_n;                   // number of source slots to sum (0: no reduce phase)
  const void* red_slots;       // bf16 [red_n][red_rows][red_ld]
  int red_rows, red_cols;
  int64_t red_ld;
  const uint32_t* red_counter; // local per-slice counters
  uint32_t* red_work;          // local per-slice work counters (zero at launch): next unit of the slot sums
  uint32_t red_target;         // counter value once every partial tile of a slice has arrived
                               // (each tile counts 4: one per epilogue warp of the sender)
  int red_slice_dim;           // 0: slice = block-cyclic row blocks (kBM), 1: column blocks (kBN)
  // the reduce phase writes to C / ldc / c_fp32 / accumulate / bias as the local epilogue does
  // ---- cross-GPU barriers ----
  int n_ranks;                 // ranks taking part (0: no barriers)
  int my_rank;
  uint32_t* entry_flags[kMaxPeers];  // rank r's entry flag array (index: source rank)
  uint32_t* exit_flags[kMaxPeers];   // rank r's exit flag array
  uint32_t epoch;              // value for this launch (monotonic per workspace)
  int exit_barrier;            // 1: wait for all peers to finish their transfers before leaving
  uint32_t* go_flag;           // local: set to epoch by CTA 0 once all peers have arrived
  uint32_t* done_counter;      // local: CTAs that finished their transfers (monotonic)
  uint32_t done_target;
  // ---- tuning of the plain (two-CTA) kernel ----
  int stages;                  // smem pipeline stages: 6 or 7
  // ---- status ----
  uint32_t* status;            // [4]: code, blockIdx, detail, detail2
  uint64_t timeout_ns;
  // ---- timeline (optional) ----
  // When non-null the launch runs the traced instantiation of the fused kernel: every CTA appends 16-byte
  // events {globaltimer ns low, high, TraceKind, argument} to its area of (trace_cap + 1) records, the first
  // of which holds the event count (zero before the launch).  16-byte aligned, gridDim.x areas.
  void* trace;
  int trace_cap;
};

// Events of the timeline: which tile, chunk or slice the argument names is given per kind.
enum TraceKind : uint32_t {
  kTraceOperandsReady = 1,   // producer: the gathered chunks that tile `arg` reads have arrived
  kTraceTileComputed = 2,    // epilogue: the accumulator of tile `arg` is complete
  kTraceTilePushed = 3,      // epilogue: the partial tile `arg` has been handed to its owner (push side)
  kTraceChunkSent = 4,       // communication warp: its share of chunk `arg` is stored and signalled everywhere
  kTraceSumBegin = 5,        // communication warp: slot sums of slice `arg` begin (all partial tiles arrived)
  kTraceSumEnd = 6,          // ... and no unit of the slice is left for this warp
};

// Launch on `stream` (grid even: CTA pairs).  Tensor maps must describe A and B with 128-byte
// swizzle and boxes {64, kBM} / {64, kBN / 2} (K-major) or {64, kBK} (MN-major).
cudaError_t launch_sm100_gemm(const CUtensorMap& tma_a, const CUtensorMap& tma_b,
                              const PushMaps& push_maps, const GemmArgs& args, int grid,
                              cudaStream_t stream);

// Two-CTA (cta_group::2) variant for plain local GEMMs (no gather / push / reduce / barriers).
// The tensor map of a K-major B must use a {64, kBN / 2} box.
cudaError_t launch_sm100_gemm2(const CUtensorMap& tma_a, const CUtensorMap& tma_b,
                               const GemmArgs& args, int grid, cudaStream_t stream);

// Builds a 2-D bf16 tensor map with 128-byte swizzle.  `inner` is the contiguous extent,
// `outer` the number of rows, `pitch_bytes` the row pitch.  Returns 0 on success.
int make_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer);

// Tensor map of an MN-major operand (stored [k_rows, mn_extent] row-major, mn_extent % 64 == 0) as
// {64 elements, k_rows, mn_extent / 64 blocks}: one box of {64, kBK, blocks_per_box} fills the
// shared-memory layout of `blocks_per_box` consecutive 64-wide blocks with ONE TMA instruction.
// Returns 0 on success (callers fall back to the 2-D map and one instruction per block).
int make_tensor_map_mn3d(CUtensorMap* map, const void* base, uint64_t mn_extent, uint64_t k_rows,
                         uint64_t pitch_bytes, uint32_t blocks_per_box);

size_t sm100_gemm_smem_bytes();

}  // namespace msb
