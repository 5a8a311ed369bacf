// netsim command line: runs one scenario or host program and prints a report (or JSON with --json).
//   netsim --scenario sendrecv --nodes 8 --topology crossbar --bytes 8388608 --link-gbs 900
//   netsim --config configs/sst_torus.ini --scenario imb --nodes 2 --bytes 1
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>

#include "config.h"

using namespace netsim;

static void usage() {
  std::puts(
      "usage: netsim [--config FILE] [--scenario NAME] [--nodes N] [--topology torus[:AxB..]|crossbar] [--bytes B]\n"
      "              [--repeat K] [--link-gbs G] [--nic-gbs G] [--hop-ns T] [--mem-gbs G] [--max-mem-reqs N]\n"
      "              [--set section.key=value]... [--dump-config] [--json]\n"
      "scenarios (NIC level, callback driven): msg write incast barrier sendrecv allgather-ring allgather-direct\n"
      "host programs (RDMA library):           rdma-hello rdma-msg rdma-write rdma-incast rdma-incast-v2\n"
      "                                        rdma-barrier rdma-sendrecv rdma-test\n"
      "message passing benchmark:              imb (PingPong PingPing Sendrecv Allreduce Reduce_scatter Allgather\n"
      "                                        Alltoall Bcast Barrier; --bytes = largest message, --repeat = iterations)");
}

static std::string json_escape(const std::string& s) {
  std::string o;
  for (char ch : s) {
    if (ch == '"' || ch == '\\') o += '\\';
    o += ch;
  }
  return o;
}

int main(int argc, char** argv) {
  ScenarioConfig c;
  bool json = false, dump = false;
  auto set = [&](const char* sec, const char* key, const std::string& v) {
    std::string err;
    if (!apply_setting(sec, key, v, c, err)) {
      std::fprintf(stderr, "netsim: %s\n", err.c_str());
      std::exit(2);
    }
  };
  for (int i = 1; i < argc; ++i) {
    auto need = [&](const char* f) {
      if (i + 1 >= argc) { std::fprintf(stderr, "%s needs a value\n", f); std::exit(2); }
      return std::string(argv[++i]);
    };
    const std::string a = argv[i];
    if (a == "--config") {
      std::string err;
      if (!load_config(need("--config"), c, err)) { std::fprintf(stderr, "netsim: %s\n", err.c_str()); return 2; }
    }
    else if (a == "--scenario") set("run", "scenario", need("--scenario"));
    else if (a == "--nodes") set("run", "nodes", need("--nodes"));
    else if (a == "--bytes") set("run", "bytes", need("--bytes"));
    else if (a == "--repeat") set("run", "repeat", need("--repeat"));
    else if (a == "--topology") set("network", "topology", need("--topology"));
    else if (a == "--link-gbs") set("network", "link_gbs", need("--link-gbs"));
    else if (a == "--nic-gbs") set("network", "nic_gbs", need("--nic-gbs"));
    else if (a == "--hop-ns") set("network", "hop_ns", need("--hop-ns"));
    else if (a == "--mem-gbs") set("memory", "gbs", need("--mem-gbs"));
    else if (a == "--max-mem-reqs") set("nic", "max_mem_reqs", need("--max-mem-reqs"));
    else if (a == "--set") {
      const std::string kv = need("--set");
      const size_t dot = kv.find('.'), eq = kv.find('=');
      if (dot == std::string::npos || eq == std::string::npos || dot > eq) {
        std::fprintf(stderr, "netsim: --set wants section.key=value\n");
        return 2;
      }
      set(kv.substr(0, dot).c_str(), kv.substr(dot + 1, eq - dot - 1).c_str(), kv.substr(eq + 1));
    }
    else if (a == "--dump-config") dump = true;
    else if (a == "--json") json = true;
    else if (a == "--help") { usage(); return 0; }
    else { std::fprintf(stderr, "unknown option %s\n", argv[i]); usage(); return 2; }
  }
  if (dump) {
    std::fputs(dump_config(c).c_str(), stdout);
    return 0;
  }
  ScenarioResult r;
  try {
    r = run_scenario(c);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "netsim: %s\n", e.what());
    return 2;
  }
  if (json) {
    std::printf("{\"scenario\": \"%s\", \"topology\": \"%s\", \"nodes\": %d, \"bytes\": %llu, \"ok\": %s, "
                "\"sim_time_us\": %.6f, \"packets\": %llu, \"events\": %llu",
                c.scenario.c_str(), c.topology.c_str(), c.nodes, (unsigned long long)c.bytes, r.ok ? "true" : "false",
                r.sim_time / 1e6, (unsigned long long)r.packets, (unsigned long long)r.events);
    for (auto& kv : r.values) std::printf(", \"%s\": %.6g", kv.first.c_str(), kv.second);
    if (!r.error.empty()) std::printf(", \"error\": \"%s\"", json_escape(r.error).c_str());
    std::printf(", \"lines\": [");
    for (size_t i = 0; i < r.lines.size(); ++i) std::printf("%s\"%s\"", i ? ", " : "", json_escape(r.lines[i]).c_str());
    std::printf("]}\n");
  } else {
    std::printf("scenario %s on %s, %d nodes, %llu bytes: %s\n", c.scenario.c_str(), c.topology.c_str(), c.nodes,
                (unsigned long long)c.bytes, r.ok ? "ok" : "FAILED");
    for (auto& l : r.lines) std::printf("%s\n", l.c_str());
    std::printf("  simulated time: %.4f us, packets: %llu, events: %llu\n", r.sim_time / 1e6,
                (unsigned long long)r.packets, (unsigned long long)r.events);
    for (auto& kv : r.values) std::printf("  %s = %g\n", kv.first.c_str(), kv.second);
    if (!r.error.empty()) std::printf("  error: %s\n", r.error.c_str());
  }
  return r.ok ? 0 : 1;
}
