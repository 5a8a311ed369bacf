// Python bindings (pybind11, no torch headers): every function takes raw device pointers
// (tensor.data_ptr()) and a stream handle (torch.cuda.current_stream().cuda_stream), so the
// extension has no ABI coupling with the PyTorch build it is used with.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "comm/p2p.h"
#include "gemm/sm100_gemm.h"
#include "ops/attention.h"
#include "ops/ops.h"

namespace py = pybind11;
using namespace msb;

namespace {

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
template <class T>
T* P(uint64_t p) { return reinterpret_cast<T*>(static_cast<uintptr_t>(p)); }
// every launcher converts its stream handle exactly once, so this also counts launches
static uint64_t g_launches = 0;
cudaStream_t S(uint64_t s) {
  ++g_launches;
  return reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(s));
}

int64_t geti(const py::dict& d, const char* k, int64_t def = 0) {
  return d.contains(k) ? d[k].cast<int64_t>() : def;
}
uint64_t getp(const py::dict& d, const char* k) {
  return d.contains(k) ? d[k].cast<uint64_t>() : 0;
}

BarrierArgs parse_barrier(const py::dict& d) {
  BarrierArgs b;
  std::memset(&b, 0, sizeof(b));
  b.n_ranks = (int)geti(d, "n_ranks");
  b.my_rank = (int)geti(d, "my_rank");
  if (b.n_ranks > kMaxPeers) throw std::runtime_error("too many ranks");
  if (b.n_ranks > 0) {
    auto ef = d["entry_flags"].cast<std::vector<uint64_t>>();
    auto xf = d["exit_flags"].cast<std::vector<uint64_t>>();
    for (int i = 0; i < b.n_ranks; ++i) {
      b.entry_flags[i] = P<uint32_t>(ef[i]);
      b.exit_flags[i] = P<uint32_t>(xf[i]);
    }
  }
  b.epoch = (uint32_t)geti(d, "epoch");
  b.go_flag = P<uint32_t>(getp(d, "go_flag"));
  b.done_counter = P<uint32_t>(getp(d, "done_counter"));
  b.done_target = (uint32_t)geti(d, "done_target");
  b.status = P<uint32_t>(getp(d, "status"));
  b.timeout_ns = (uint64_t)geti(d, "timeout_ns", 5000000000LL);
  return b;
}

// Row exchange descriptor from a dict (None or empty: no exchange).  Keys: n, me, dst[n], slots,
// stride, counter[n], my_counter, target, timeout_ns, status.
struct ParsedExchange {
  RowExchange ex;
  bool on;
  const RowExchange* ptr() const { return on ? &ex : nullptr; }
};
ParsedExchange parse_exchange(const py::object& o) {
  ParsedExchange r;
  std::memset(&r.ex, 0, sizeof(r.ex));
  r.on = false;
  if (o.is_none()) return r;
  py::dict d = o.cast<py::dict>();
  const int n = (int)geti(d, "n");
  if (n <= 1) return r;
  if (n > kExMaxPeers) throw std::runtime_error("row exchange: too many GPUs in the group");
  r.ex.n = n;
  r.ex.me = (int)geti(d, "me");
  auto dst = d["dst"].cast<std::vector<uint64_t>>();
  auto cnt = d["counter"].cast<std::vector<uint64_t>>();
  if ((int)dst.size() != n || (int)cnt.size() != n || r.ex.me < 0 || r.ex.me >= n)
    throw std::runtime_error("row exchange: need one slot area and one counter per GPU of the group");
  for (int i = 0; i < n; ++i) {
    if (dst[i] == 0 || (dst[i] & 15) || cnt[i] == 0) throw std::runtime_error("row exchange: bad pointer");
    r.ex.dst[i] = P<float>(dst[i]);
    r.ex.counter[i] = P<uint32_t>(cnt[i]);
  }
  r.ex.slots = P<const float>(getp(d, "slots"));
  r.ex.stride = geti(d, "stride");
  r.ex.my_counter = P<const uint32_t>(getp(d, "my_counter"));
  r.ex.target = (uint32_t)geti(d, "target");
  r.ex.timeout_ns = (uint64_t)geti(d, "timeout_ns", 20000000000LL);
  r.ex.status = P<uint32_t>(getp(d, "status"));
  if (r.ex.slots == nullptr || r.ex.my_counter == nullptr || r.ex.status == nullptr || r.ex.stride <= 0)
    throw std::runtime_error("row exchange: slots, my_counter, status and stride are required");
  r.on = true;
  return r;
}

// ---------------------------------------------------------------------------------------
// GEMM
// ---------------------------------------------------------------------------------------
void gemm_run(const py::dict& d) {
  GemmArgs a;
  std::memset(&a, 0, sizeof(a));
  a.M = (int)geti(d, "M");
  a.N = (int)geti(d, "N");
  a.K = (int)geti(d, "K");
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) throw std::runtime_error("gemm: empty problem");
  a.a_mn_major = (int)geti(d, "a_mn_major");
  a.b_mn_major = (int)geti(d, "b_mn_major");
  const uint64_t A = getp(d, "A"), B = getp(d, "B");
  const int64_t lda = geti(d, "lda"), ldb = geti(d, "ldb");
  if ((lda % 8) || (ldb % 8) || (A & 15) || (B & 15))
    throw std::runtime_error("gemm: operands need 16-byte aligned bases and pitches");
  a.C = P<void>(getp(d, "C"));
  a.ldc = geti(d, "ldc");
  a.c_fp32 = (int)geti(d, "c_fp32");
  a.accumulate = (int)geti(d, "accumulate");
  a.bias = P<void>(getp(d, "bias"));
  a.act = (int)geti(d, "act");
  a.C_pre = P<void>(getp(d, "C_pre"));
  if (a.ldc % 8) throw std::runtime_error("gemm: ldc must be a multiple of 8");
  a.tiles_m = (a.M + 2 * kBM - 1) / (2 * kBM);   // 256-row cluster tiles
  a.tiles_n = (a.N + kBN - 1) / kBN;
  a.slice_dim = (int)geti(d, "slice_dim");
  a.n_slices = (int)geti(d, "n_slices", 1);
  a.group = (int)geti(d, "group", 8);
  const int tiles_s = a.slice_dim == 0 ? a.tiles_m : a.tiles_n;
  a.cyc = (int)geti(d, "cyc", 1);
  if (a.cyc < 1) a.cyc = 1;
  if (a.n_slices < 1 || tiles_s % (a.n_slices * a.cyc) != 0)
    throw std::runtime_error("gemm: n_slices must divide the tile count of the sliced dimension");
  if (a.group < 1) a.group = 1;
  a.stages = (int)geti(d, "stages", 7);
  a.rot = (int)geti(d, "rot", 0);
  if (a.rot < 0 || a.rot >= tiles_s / a.n_slices) a.rot = 0;
  if (geti(d, "no_tiles")) a.tiles_m = 0;  // reduce phase only
  // gather side
  a.jobs = P<const PushJob>(getp(d, "jobs"));
  a.chunks = P<const ChunkDesc>(getp(d, "chunks"));
  a.skip_comm = (int)geti(d, "skip_comm");
  a.gather_src[0] = P<const char>(getp(d, "gather_src0"));
  a.gather_src[1] = P<const char>(getp(d, "gather_src1"));
  a.n_chunks = (int)geti(d, "n_chunks");
  a.chunk_flags = P<uint32_t>(getp(d, "chunk_flags"));
  a.a_flag_mode = (int)geti(d, "a_flag_mode");
  a.a_flag_base = (int)geti(d, "a_flag_base");
  a.a_flag_count = (int)geti(d, "a_flag_count");
  a.b_flag_mode = (int)geti(d, "b_flag_mode");
  a.b_flag_base = (int)geti(d, "b_flag_base");
  a.b_flag_count = (int)geti(d, "b_flag_count");
  a.a_flag_target = (uint32_t)geti(d, "a_flag_target", 0);
  a.b_flag_target = (uint32_t)geti(d, "b_flag_target", 0);
  if ((a.a_flag_mode != 0 && a.a_flag_mode != 3 && a.a_flag_target == 0) ||
      (a.b_flag_mode != 0 && a.b_flag_mode != 3 && a.b_flag_target == 0))
    throw std::runtime_error("gemm: a gathered operand needs its flag target");
  a.b_nchunk = (int)geti(d, "b_nchunk", 1);
  if (a.b_nchunk < 1) a.b_nchunk = 1;
  a.a_kpanel = (int)geti(d, "a_kpanel", 1);
  a.b_kpanel = (int)geti(d, "b_kpanel", 1);
  a.kp_target = (uint32_t)geti(d, "kp_target", 0);
  a.k_rot = (int)geti(d, "k_rot", 0);
  if (a.a_kpanel < 1 || a.b_kpanel < 1 || a.k_rot < 0 || a.k_rot >= std::max<int64_t>(1, (a.K + kBK - 1) / kBK))
    throw std::runtime_error("gemm: bad K-panel schedule");
  if ((a.a_flag_mode == 3 || a.b_flag_mode == 3) && a.K % kBK != 0)
    throw std::runtime_error("gemm: the K-panel schedule needs K to be a multiple of 64");
  // push side
  a.push_n = (int)geti(d, "push_n");
  if (a.push_n > kMaxPeers) throw std::runtime_error("gemm: too many owners");
  a.push_dim = (int)geti(d, "push_dim");
  a.push_extent = (int)geti(d, "push_extent", 1);
  a.push_bufs = (int)geti(d, "push_bufs", 1);
  a.push_mode = (int)geti(d, "push_mode", 0);
  a.push_ld = geti(d, "push_ld");
  if (a.push_n > 0) {
    auto pb = d["push_base"].cast<std::vector<uint64_t>>();
    auto pc = d["push_counter"].cast<std::vector<uint64_t>>();
    for (int i = 0; i < a.push_n; ++i) {
      a.push_base[i] = P<void>(pb[i]);
      a.push_counter[i] = P<uint32_t>(pc[i]);
    }
    const int tile = a.push_dim == 0 ? 2 * kBM : kBN;
    if (a.push_extent % tile != 0 || a.push_ld % 8 != 0 || a.M % (2 * kBM) != 0 || a.N % kBN != 0)
      throw std::runtime_error("gemm: owner extent must be a multiple of the tile size");
  }
  a.red_n = (int)geti(d, "red_n");
  a.red_slots = P<const void>(getp(d, "red_slots"));
  a.red_rows = (int)geti(d, "red_rows");
  a.red_cols = (int)geti(d, "red_cols");
  a.red_ld = geti(d, "red_ld");
  a.red_counter = P<const uint32_t>(getp(d, "red_counter"));
  a.red_target = (uint32_t)geti(d, "red_target");
  a.red_work = P<uint32_t>(getp(d, "red_work"));
  if (a.red_n > 0 && a.red_work == nullptr) throw std::runtime_error("gemm: the reduce phase needs its work counters");
  a.red_slice_dim = (int)geti(d, "red_slice_dim");
  if (a.red_n > 0) {
    const int rt = a.red_slice_dim == 0 ? (a.red_rows + 2 * kBM - 1) / (2 * kBM) : (a.red_cols + kBN - 1) / kBN;
    if (rt % (a.n_slices * a.cyc) != 0 || a.red_cols % 8 != 0 || a.red_ld % 8 != 0)
      throw std::runtime_error("gemm: reduce phase shape not divisible by the slice count");
  }
  // barriers
  BarrierArgs b = parse_barrier(d);
  a.n_ranks = b.n_ranks;
  a.my_rank = b.my_rank;
  for (int i = 0; i < kMaxPeers; ++i) {
    a.entry_flags[i] = b.entry_flags[i];
    a.exit_flags[i] = b.exit_flags[i];
  }
  a.epoch = b.epoch;
  a.exit_barrier = (int)geti(d, "exit_barrier");
  a.go_flag = b.go_flag;
  a.done_counter = b.done_counter;
  a.done_target = b.done_target;
  a.status = b.status;
  a.timeout_ns = b.timeout_ns;
  if (a.status == nullptr) throw std::runtime_error("gemm: status pointer required");
  a.trace = P<void>(getp(d, "trace"));
  a.trace_cap = (int)geti(d, "trace_cap", 0);
  if (a.trace != nullptr && (a.trace_cap <= 0 || (getp(d, "trace") & 15)))
    throw std::runtime_error("gemm: the timeline buffer needs trace_cap > 0 and 16-byte alignment");

  CUtensorMap ta, tb;
  int r;
  const bool try3d = geti(d, "map3d", 1) != 0;
  if (!a.a_mn_major) r = make_tensor_map_2d(&ta, P<void>(A), a.K, a.M, lda * 2, kBK, kBM);
  else if (try3d && make_tensor_map_mn3d(&ta, P<void>(A), a.M, a.K, lda * 2, kBM / 64) == 0) { r = 0; a.a_map3d = 1; }
  else r = make_tensor_map_2d(&ta, P<void>(A), a.M, a.K, lda * 2, 64, kBK);
  if (r != 0) throw std::runtime_error("gemm: tensor map for A failed, code " + std::to_string(r));
  const bool plain = a.n_chunks == 0 && a.n_ranks == 0 && a.red_n == 0 && a.push_n == 0 && a.tiles_m > 0;
  const bool pair = plain && geti(d, "two_cta", 1) != 0;
  if (!a.b_mn_major) r = make_tensor_map_2d(&tb, P<void>(B), a.K, a.N, ldb * 2, kBK, kBN / 2);
  else if (try3d && make_tensor_map_mn3d(&tb, P<void>(B), a.N, a.K, ldb * 2, kBN / 128) == 0) { r = 0; a.b_map3d = 1; }
  else r = make_tensor_map_2d(&tb, P<void>(B), a.N, a.K, ldb * 2, 64, kBK);
  if (r != 0) throw std::runtime_error("gemm: tensor map for B failed, code " + std::to_string(r));

  int grid = (int)geti(d, "grid", 148);
  const int ntiles = a.tiles_m * a.tiles_n;
  const bool needs_all = a.n_chunks > 0 || a.n_ranks > 0 || a.red_n > 0;
  if (!needs_all && grid > 2 * ntiles) grid = 2 * ntiles;
  grid &= ~1;
  if (grid < 2) grid = 2;
  if (pair) {
    const int clusters = ((a.M + 2 * kBM - 1) / (2 * kBM)) * a.tiles_n;
    int g2 = (int)geti(d, "grid", 148) & ~1;
    if (g2 > 2 * clusters) g2 = 2 * clusters;
    check(launch_sm100_gemm2(ta, tb, a, g2, S(getp(d, "stream"))), "sm100_gemm2 launch");
    return;
  }
  static PushMaps pm;   // only the first push_n entries are read by the kernel
  if (a.push_n > 0) {
    const uint64_t rows = (uint64_t)geti(d, "push_rows");
    if (rows == 0) throw std::runtime_error("gemm: push_rows (rows of an owner's slot) required");
    for (int i = 0; i < a.push_n; ++i) {
      r = make_tensor_map_2d(&pm.m[i], a.push_base[i], (uint64_t)a.push_ld, rows, (uint64_t)a.push_ld * 2, 64, 32);
      if (r != 0) throw std::runtime_error("gemm: tensor map for an owner's slot failed, code " + std::to_string(r));
    }
  }
  check(launch_sm100_gemm(ta, tb, pm, a, grid, S(getp(d, "stream"))), "sm100_gemm launch");
}

// ---------------------------------------------------------------------------------------
// runtime: IPC-shared device memory, host-mapped status words
// ---------------------------------------------------------------------------------------
py::tuple symm_alloc(size_t bytes) {
  void* p = nullptr;
  check(cudaMalloc(&p, bytes), "cudaMalloc(symmetric heap)");
  cudaIpcMemHandle_t h;
  check(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle");
  return py::make_tuple((uint64_t)(uintptr_t)p,
                        py::bytes(reinterpret_cast<const char*>(&h), sizeof(h)));
}
uint64_t symm_open(const py::bytes& handle) {
  std::string s = handle;
  if (s.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("bad IPC handle size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, s.data(), sizeof(h));
  void* p = nullptr;
  check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return (uint64_t)(uintptr_t)p;
}
void symm_close(uint64_t p) { check(cudaIpcCloseMemHandle(P<void>(p)), "cudaIpcCloseMemHandle"); }
void symm_free(uint64_t p) { check(cudaFree(P<void>(p)), "cudaFree"); }

py::tuple status_alloc() {
  void* h = nullptr;
  check(cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable), "cudaHostAlloc");
  std::memset(h, 0, 64);
  void* dptr = nullptr;
  check(cudaHostGetDevicePointer(&dptr, h, 0), "cudaHostGetDevicePointer");
  return py::make_tuple((uint64_t)(uintptr_t)h, (uint64_t)(uintptr_t)dptr);
}
py::tuple status_read(uint64_t host_ptr) {
  volatile uint32_t* s = P<volatile uint32_t>(host_ptr);
  return py::make_tuple(s[0], s[1], s[2], s[3]);
}
void status_clear(uint64_t host_ptr) { std::memset(P<void>(host_ptr), 0, 64); }

void memset_zero(uint64_t ptr, size_t bytes, uint64_t stream) {
  check(cudaMemsetAsync(P<void>(ptr), 0, bytes,
                        reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(stream))),
        "cudaMemsetAsync");
}

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "meshslice_b200 native kernels (sm_100a)";
  m.attr("BM") = kBM;
  m.attr("BN") = kBN;
  m.attr("BK") = kBK;
  m.attr("MAX_PEERS") = kMaxPeers;
  m.attr("COPY_JOB_BYTES") = (int)sizeof(CopyJob);
  m.attr("AUX_WARPS") = (int)kAuxWarps;   // communication warps per CTA: each bumps a chunk flag once
  m.attr("PUSH_JOB_BYTES") = (int)sizeof(PushJob);
  m.attr("CHUNK_DESC_BYTES") = (int)sizeof(ChunkDesc);

  m.def("gemm_run", &gemm_run, "persistent tcgen05 GEMM with optional fused gather / push");
  m.def("symm_alloc", &symm_alloc);
  m.def("symm_open", &symm_open);
  m.def("symm_close", &symm_close);
  m.def("symm_free", &symm_free);
  m.def("status_alloc", &status_alloc);
  m.def("status_read", &status_read);
  m.def("status_clear", &status_clear);
  m.def("memset_zero", &memset_zero);
  m.def("launch_count", []() { return g_launches; }, "kernel launches issued by this module so far");

  m.def("p2p_copy", [](uint64_t jobs, int n_jobs, const py::dict& bar, int grid, uint64_t stream) {
    check(p2p_copy(P<const CopyJob>(jobs), n_jobs, parse_barrier(bar), grid, S(stream)), "p2p_copy");
  });
  m.def("p2p_reduce", [](std::vector<uint64_t> src, int64_t src_pitch, uint64_t out, int64_t out_pitch,
                         int rows, int cols, const py::dict& bar, int grid, uint64_t stream) {
    ReduceArgs r;
    std::memset(&r, 0, sizeof(r));
    if ((int)src.size() > kMaxPeers) throw std::runtime_error("p2p_reduce: too many sources");
    r.n_src = (int)src.size();
    for (int i = 0; i < r.n_src; ++i) r.src[i] = P<const void>(src[i]);
    r.src_pitch = src_pitch;
    r.out = P<void>(out);
    r.out_pitch = out_pitch;
    r.rows = rows;
    r.cols = cols;
    check(p2p_reduce(r, parse_barrier(bar), grid, S(stream)), "p2p_reduce");
  });
  m.def("p2p_barrier", [](const py::dict& bar, uint64_t stream) {
    check(p2p_barrier(parse_barrier(bar), S(stream)), "p2p_barrier");
  });
  m.def("bounded_wait_probe", [](uint64_t flag, uint32_t target, uint64_t timeout_ns, uint64_t status,
                                 uint64_t stream) {
    check(bounded_wait_probe(P<const uint32_t>(flag), target, timeout_ns, P<uint32_t>(status), S(stream)),
          "bounded_wait_probe");
  });

  // ---- ops ----
  m.def("ln_fwd", [](int mode, uint64_t x, uint64_t res, uint64_t h_out, uint64_t y, uint64_t gamma,
                     uint64_t beta, uint64_t stats, uint64_t mean_rstd, int rows, int cols,
                     int total_cols, float eps, uint64_t stream, py::object exch) {
    const ParsedExchange e = parse_exchange(exch);
    check(ln_fwd(mode, P<void>(x), P<void>(res), P<void>(h_out), P<void>(y), P<void>(gamma),
                 P<void>(beta), P<float>(stats), P<float>(mean_rstd), rows, cols, total_cols, eps,
                 S(stream), e.ptr()), "ln_fwd");
  }, py::arg("mode"), py::arg("x"), py::arg("res"), py::arg("h_out"), py::arg("y"), py::arg("gamma"),
     py::arg("beta"), py::arg("stats"), py::arg("mean_rstd"), py::arg("rows"), py::arg("cols"),
     py::arg("total_cols"), py::arg("eps"), py::arg("stream"), py::arg("exch") = py::none());
  m.def("ln_bwd", [](int mode, uint64_t dy, uint64_t h, uint64_t gamma, uint64_t mean_rstd,
                     uint64_t dres, uint64_t dx, uint64_t stats, uint64_t dgamma, uint64_t dbeta,
                     int rows, int cols, int total_cols, uint64_t stream, py::object exch) {
    const ParsedExchange e = parse_exchange(exch);
    check(ln_bwd(mode, P<void>(dy), P<void>(h), P<void>(gamma), P<float>(mean_rstd), P<void>(dres),
                 P<void>(dx), P<float>(stats), P<float>(dgamma), P<float>(dbeta), rows, cols,
                 total_cols, S(stream), e.ptr()), "ln_bwd");
  }, py::arg("mode"), py::arg("dy"), py::arg("h"), py::arg("gamma"), py::arg("mean_rstd"), py::arg("dres"),
     py::arg("dx"), py::arg("stats"), py::arg("dgamma"), py::arg("dbeta"), py::arg("rows"), py::arg("cols"),
     py::arg("total_cols"), py::arg("stream"), py::arg("exch") = py::none());
  m.def("ln_grid", &ln_grid, py::arg("backward"), py::arg("rows"), py::arg("cols") = 0,
        "CTAs of the LayerNorm kernels for a row count and local width (0: forward, 1: backward)");
  m.def("ce_grid", &ce_grid, "CTAs of the cross-entropy kernels for a row count");
  m.def("gelu_fwd", [](uint64_t x, uint64_t y, int64_t n, uint64_t stream) {
    check(gelu_fwd(P<void>(x), P<void>(y), n, S(stream)), "gelu_fwd");
  });
  m.def("gelu_bwd", [](uint64_t dy, uint64_t x, uint64_t dx, int64_t n, uint64_t stream) {
    check(gelu_bwd(P<void>(dy), P<void>(x), P<void>(dx), n, S(stream)), "gelu_bwd");
  });
  m.def("add_bf16", [](uint64_t a, uint64_t b, uint64_t o, int64_t n, uint64_t stream) {
    check(add_bf16(P<void>(a), P<void>(b), P<void>(o), n, S(stream)), "add_bf16");
  });
  m.def("cast_f32_to_bf16", [](uint64_t in, uint64_t out, int64_t n, int accumulate, uint64_t stream) {
    check(cast_f32_to_bf16(P<float>(in), P<void>(out), n, accumulate, S(stream)), "cast_f32_to_bf16");
  });
  m.def("adamw_step", [](uint64_t param, uint64_t master, uint64_t mm, uint64_t vv, uint64_t grad,
                         int grad_fp32, int64_t n, float lr, float b1, float b2, float eps, float wd,
                         float bc1, float bc2, uint64_t grad_scale, uint64_t stream) {
    check(adamw_step(P<void>(param), P<float>(master), P<float>(mm), P<float>(vv), P<void>(grad),
                     grad_fp32, n, lr, b1, b2, eps, wd, bc1, bc2, P<float>(grad_scale), S(stream)),
          "adamw_step");
  });
  m.def("sumsq", [](uint64_t x, int is_fp32, int64_t n, uint64_t out, uint64_t stream) {
    check(sumsq(P<void>(x), is_fp32, n, P<float>(out), S(stream)), "sumsq");
  });
  m.def("ce_partial", [](uint64_t logits, int64_t ld, uint64_t targets, int rows, int cols,
                         int col_offset, int vocab, uint64_t row_max, uint64_t row_sumexp,
                         uint64_t tgt_logit, uint64_t stream, py::object exch) {
    const ParsedExchange e = parse_exchange(exch);
    check(ce_partial(P<void>(logits), ld, P<int64_t>(targets), rows, cols, col_offset, vocab,
                     P<float>(row_max), P<float>(row_sumexp), P<float>(tgt_logit), S(stream), e.ptr()),
          "ce_partial");
  }, py::arg("logits"), py::arg("ld"), py::arg("targets"), py::arg("rows"), py::arg("cols"),
     py::arg("col_offset"), py::arg("vocab"), py::arg("row_max"), py::arg("row_sumexp"), py::arg("tgt_logit"),
     py::arg("stream"), py::arg("exch") = py::none());
  m.def("ce_grad", [](uint64_t logits, int64_t ld, uint64_t targets, int rows, int cols,
                      int col_offset, int vocab, uint64_t gmax, uint64_t gsum, float scale,
                      uint64_t stream, uint64_t row_loss, py::object exch) {
    const ParsedExchange e = parse_exchange(exch);
    check(ce_grad(P<void>(logits), ld, P<int64_t>(targets), rows, cols, col_offset, vocab,
                  P<float>(gmax), P<float>(gsum), scale, S(stream), P<float>(row_loss), e.ptr()), "ce_grad");
  }, py::arg("logits"), py::arg("ld"), py::arg("targets"), py::arg("rows"), py::arg("cols"),
     py::arg("col_offset"), py::arg("vocab"), py::arg("gmax"), py::arg("gsum"), py::arg("scale"),
     py::arg("stream"), py::arg("row_loss") = 0, py::arg("exch") = py::none());
  m.def("embedding_fwd", [](uint64_t tokens, uint64_t tok, uint64_t pos, uint64_t out, int n_tokens,
                            int seq, int cols, uint64_t stream) {
    check(embedding_fwd(P<int64_t>(tokens), P<void>(tok), P<void>(pos), P<void>(out), n_tokens, seq,
                        cols, S(stream)), "embedding_fwd");
  });
  m.def("embedding_bwd", [](uint64_t tokens, uint64_t dout, uint64_t dtok, uint64_t dpos,
                            int n_tokens, int seq, int cols, uint64_t stream) {
    check(embedding_bwd(P<int64_t>(tokens), P<void>(dout), P<float>(dtok), P<float>(dpos), n_tokens,
                        seq, cols, S(stream)), "embedding_bwd");
  });
  m.def("attention_fwd", [](uint64_t qkv, uint64_t out, uint64_t lse, int batch, int seq, int heads,
                            int causal, float scale, uint64_t status, uint64_t stream) {
    check(attention_fwd(P<void>(qkv), P<void>(out), P<float>(lse), batch, seq, heads, causal, scale,
                        P<uint32_t>(status), S(stream)), "attention_fwd");
  });
  m.def("attention_bwd", [](uint64_t qkv, uint64_t out, uint64_t dout, uint64_t lse, uint64_t dqkv,
                            uint64_t dq_acc, uint64_t delta, int batch, int seq, int heads, int causal,
                            float scale, uint64_t status, uint64_t stream) {
    check(attention_bwd(P<void>(qkv), P<void>(out), P<void>(dout), P<float>(lse), P<void>(dqkv),
                        P<float>(dq_acc), P<float>(delta), batch, seq, heads, causal, scale,
                        P<uint32_t>(status), S(stream)), "attention_bwd");
  });
}
