// netsim command line: runs one scenario and prints a small report (or JSON with --json).
//   netsim --scenario sendrecv --nodes 8 --topology crossbar --bytes 8388608 --link-gbs 900
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>

#include "scenarios.h"

using namespace netsim;

static void usage() {
  std::puts("usage: netsim [--scenario msg|write|incast|barrier|sendrecv|allgather-ring|allgather-direct]\n"
            "              [--nodes N] [--topology torus[:AxB..]|crossbar] [--bytes B] [--repeat K]\n"
            "              [--link-gbs G] [--nic-gbs G] [--hop-ns T] [--mem-gbs G] [--max-mem-reqs N] [--json]");
}

int main(int argc, char** argv) {
  ScenarioConfig c;
  bool json = false;
  for (int i = 1; i < argc; ++i) {
    auto need = [&](const char* f) {
      if (i + 1 >= argc) { std::fprintf(stderr, "%s needs a value\n", f); std::exit(2); }
      return argv[++i];
    };
    if (!std::strcmp(argv[i], "--scenario")) c.scenario = need("--scenario");
    else if (!std::strcmp(argv[i], "--nodes")) c.nodes = std::atoi(need("--nodes"));
    else if (!std::strcmp(argv[i], "--topology")) c.topology = need("--topology");
    else if (!std::strcmp(argv[i], "--bytes")) c.bytes = std::strtoull(need("--bytes"), nullptr, 10);
    else if (!std::strcmp(argv[i], "--repeat")) c.repeat = std::atoi(need("--repeat"));
    else if (!std::strcmp(argv[i], "--link-gbs")) c.net.link_bw = std::atof(need("--link-gbs")) * 1e9;
    else if (!std::strcmp(argv[i], "--nic-gbs")) c.net.nic_bw = std::atof(need("--nic-gbs")) * 1e9;
    else if (!std::strcmp(argv[i], "--hop-ns")) c.net.link_latency = (Time)(std::atof(need("--hop-ns")) * kNs);
    else if (!std::strcmp(argv[i], "--mem-gbs")) c.nic.mem_bw = std::atof(need("--mem-gbs")) * 1e9;
    else if (!std::strcmp(argv[i], "--max-mem-reqs")) c.nic.max_mem_reqs = std::atoi(need("--max-mem-reqs"));
    else if (!std::strcmp(argv[i], "--json")) json = true;
    else if (!std::strcmp(argv[i], "--help")) { usage(); return 0; }
    else { std::fprintf(stderr, "unknown option %s\n", argv[i]); usage(); return 2; }
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
    if (!r.error.empty()) std::printf(", \"error\": \"%s\"", r.error.c_str());
    std::printf("}\n");
  } else {
    std::printf("scenario %s on %s, %d nodes, %llu bytes: %s\n", c.scenario.c_str(), c.topology.c_str(), c.nodes,
                (unsigned long long)c.bytes, r.ok ? "ok" : "FAILED");
    std::printf("  simulated time: %.4f us, packets: %llu, events: %llu\n", r.sim_time / 1e6,
                (unsigned long long)r.packets, (unsigned long long)r.events);
    for (auto& kv : r.values) std::printf("  %s = %g\n", kv.first.c_str(), kv.second);
    if (!r.error.empty()) std::printf("  error: %s\n", r.error.c_str());
  }
  return r.ok ? 0 : 1;
}
