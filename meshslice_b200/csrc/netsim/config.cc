// netsim: ini reader for system descriptions (see config.h).
#include "config.h"

#include <cstdlib>
#include <fstream>
#include <sstream>

namespace netsim {

namespace {

std::string trim(const std::string& s) {
  size_t a = s.find_first_not_of(" \t\r\n"), b = s.find_last_not_of(" \t\r\n");
  return a == std::string::npos ? "" : s.substr(a, b - a + 1);
}

bool number(const std::string& v, double& out) {
  char* end = nullptr;
  out = std::strtod(v.c_str(), &end);
  return end != v.c_str() && *end == '\0';
}

void resolve_memory(ScenarioConfig& cfg) {   // [memory] -> the NIC's DMA latency and bandwidth
  const MemoryParams& m = cfg.memory;
  cfg.nic.mem_latency = (Time)(m.latency_ns * kNs);
  cfg.nic.mem_bw = (m.kind == "hbm" ? m.channels * m.channel_gbs : m.gbs) * 1e9;
}

}  // namespace

bool apply_setting(const std::string& sec, const std::string& key, const std::string& val, ScenarioConfig& c,
                   std::string& err) {
  double x = 0;
  const bool is_num = number(val, x);
  auto need_num = [&]() {
    if (!is_num) err = "'" + val + "' is not a number";
    return is_num;
  };
  auto positive = [&]() {
    if (!need_num()) return false;
    if (x <= 0) err = key + " must be positive";
    return x > 0;
  };
  if (sec == "run") {
    if (key == "scenario") { c.scenario = val; return true; }
    if (key == "nodes") { if (!positive()) return false; c.nodes = (int)x; return true; }
    if (key == "bytes") { if (!need_num() || x < 0) { err = "bytes must be a non-negative number"; return false; } c.bytes = (uint64_t)x; return true; }
    if (key == "repeat") { if (!positive()) return false; c.repeat = (int)x; return true; }
  } else if (sec == "network") {
    if (key == "topology") { c.topology = val; return true; }
    if (key == "link_gbs") { if (!positive()) return false; c.net.link_bw = x * 1e9; return true; }
    if (key == "nic_gbs") { if (!positive()) return false; c.net.nic_bw = x * 1e9; return true; }
    if (key == "hop_ns") { if (!need_num()) return false; c.net.link_latency = (Time)(x * kNs); return true; }
    if (key == "router_ns") { if (!need_num()) return false; c.net.router_latency = (Time)(x * kNs); return true; }
    if (key == "flit_bytes") { if (!positive()) return false; c.net.flit_bytes = (uint32_t)x; return true; }
  } else if (sec == "nic") {
    if (key == "clock_ns") { if (!positive()) return false; c.nic.clock = (Time)(x * kNs); return true; }
    if (key == "cmd_q_size") { if (!positive()) return false; c.nic.cmd_q_size = (uint32_t)x; return true; }
    if (key == "max_mem_reqs") { if (!positive()) return false; c.nic.max_mem_reqs = (uint32_t)x; return true; }
    if (key == "mem_req_bytes") { if (!positive()) return false; c.nic.mem_req_bytes = (uint32_t)x; return true; }
    if (key == "barrier_degree") { if (!positive() || x < 2) { err = "barrier_degree must be at least 2"; return false; } c.nic.barrier_degree = (uint32_t)x; return true; }
    if (key == "out_q_depth") { if (!positive()) return false; c.nic.out_q_depth = (uint32_t)x; return true; }
    if (key == "send_ready_depth") { if (!positive()) return false; c.nic.send_ready_depth = (uint32_t)x; return true; }
    if (key == "host_cmd_ns") { if (!need_num()) return false; c.nic.host_cmd_latency = (Time)(x * kNs); return true; }
    if (key == "host_poll_ns") { if (!need_num()) return false; c.nic.host_poll_latency = (Time)(x * kNs); return true; }
  } else if (sec == "memory") {
    if (key == "kind") {
      if (val != "simple" && val != "hbm") { err = "memory kind must be 'simple' or 'hbm'"; return false; }
      c.memory.kind = val;
    } else if (key == "channels") { if (!positive()) return false; c.memory.channels = x; }
    else if (key == "channel_gbs") { if (!positive()) return false; c.memory.channel_gbs = x; }
    else if (key == "latency_ns") { if (!need_num()) return false; c.memory.latency_ns = x; }
    else if (key == "gbs") { if (!positive()) return false; c.memory.gbs = x; }
    else { err = "unknown key '" + key + "' in [memory]"; return false; }
    resolve_memory(c);
    return true;
  } else if (sec == "host") {
    if (key == "call_overhead_ns") { if (!need_num()) return false; c.host.call_overhead = (Time)(x * kNs); return true; }
  } else if (sec == "mpi") {
    if (key == "eager_limit") { if (!positive()) return false; c.mpi.eager_limit = (uint32_t)x; return true; }
    if (key == "posted_recvs") { if (!positive()) return false; c.mpi.posted_recvs = (uint32_t)x; return true; }
    if (key == "cq_entries") { if (!positive()) return false; c.mpi.cq_entries = (uint32_t)x; return true; }
    if (key == "copy_gbs") { if (!positive()) return false; c.mpi.copy_gbs = x; return true; }
    if (key == "reduce_gbs") { if (!positive()) return false; c.mpi.reduce_gbs = x; return true; }
    if (key == "coll_overhead_ns") { if (!need_num()) return false; c.mpi.coll_overhead = (Time)(x * kNs); return true; }
    if (key == "match_ns") { if (!need_num()) return false; c.mpi.match_overhead = (Time)(x * kNs); return true; }
  } else {
    err = "unknown section [" + sec + "]";
    return false;
  }
  if (err.empty()) err = "unknown key '" + key + "' in [" + sec + "]";
  return false;
}

bool load_config(const std::string& path, ScenarioConfig& cfg, std::string& error) {
  std::ifstream in(path);
  if (!in) {
    error = path + ": cannot open";
    return false;
  }
  std::string line, section;
  int no = 0;
  while (std::getline(in, line)) {
    ++no;
    const size_t hash = line.find_first_of("#;");
    if (hash != std::string::npos) line.erase(hash);
    line = trim(line);
    if (line.empty()) continue;
    auto fail = [&](const std::string& m) {
      error = path + ":" + std::to_string(no) + ": " + m;
      return false;
    };
    if (line.front() == '[') {
      if (line.back() != ']') return fail("unterminated section header");
      section = trim(line.substr(1, line.size() - 2));
      continue;
    }
    const size_t eq = line.find('=');
    if (eq == std::string::npos) return fail("expected key = value");
    if (section.empty()) return fail("setting outside of a section");
    std::string err;
    if (!apply_setting(section, trim(line.substr(0, eq)), trim(line.substr(eq + 1)), cfg, err)) return fail(err);
  }
  return true;
}

std::string dump_config(const ScenarioConfig& c) {
  std::ostringstream o;
  o << "[run]\nscenario = " << c.scenario << "\nnodes = " << c.nodes << "\nbytes = " << c.bytes << "\nrepeat = " << c.repeat
    << "\n[network]\ntopology = " << c.topology << "\nlink_gbs = " << c.net.link_bw / 1e9 << "\nnic_gbs = " << c.net.nic_bw / 1e9
    << "\nhop_ns = " << c.net.link_latency / (double)kNs << "\nrouter_ns = " << c.net.router_latency / (double)kNs
    << "\nflit_bytes = " << c.net.flit_bytes << "\n[nic]\nclock_ns = " << c.nic.clock / (double)kNs
    << "\ncmd_q_size = " << c.nic.cmd_q_size << "\nmax_mem_reqs = " << c.nic.max_mem_reqs << "\nmem_req_bytes = " << c.nic.mem_req_bytes
    << "\nbarrier_degree = " << c.nic.barrier_degree << "\nout_q_depth = " << c.nic.out_q_depth
    << "\nsend_ready_depth = " << c.nic.send_ready_depth << "\nhost_cmd_ns = " << c.nic.host_cmd_latency / (double)kNs
    << "\nhost_poll_ns = " << c.nic.host_poll_latency / (double)kNs << "\n[memory]\nkind = " << c.memory.kind << "\ngbs = " << c.memory.gbs << "\nchannels = " << c.memory.channels
    << "\nchannel_gbs = " << c.memory.channel_gbs << "\nlatency_ns = " << c.memory.latency_ns << "\n[host]\ncall_overhead_ns = " << c.host.call_overhead / (double)kNs
    << "\n[mpi]\neager_limit = " << c.mpi.eager_limit << "\nposted_recvs = " << c.mpi.posted_recvs << "\ncq_entries = " << c.mpi.cq_entries
    << "\ncopy_gbs = " << c.mpi.copy_gbs << "\nreduce_gbs = " << c.mpi.reduce_gbs << "\nmatch_ns = " << c.mpi.match_overhead / (double)kNs << "\ncoll_overhead_ns = " << c.mpi.coll_overhead / (double)kNs
    << "\n";
  return o.str();
}

}  // namespace netsim
