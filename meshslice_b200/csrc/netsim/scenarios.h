// netsim: scripted scenarios (the reference's RDMA test programs msg / write / incast / barrier /
// sendrecv, tests/app/rdma/*.c, as event-driven scripts) and simple collectives built on the
// one-sided API, used to produce latency / bandwidth curves comparable to a collectives sweep.
#pragma once
#include <map>
#include <string>

#include "mpi.h"

namespace netsim {

// Host memory as the NIC's DMA engine sees it: one latency and either a flat bandwidth ('simple')
// or channels x per-channel bandwidth ('hbm', the reference's hbmmemory.py / hbmsystem.ini variant).
struct MemoryParams {
  std::string kind = "simple";
  double gbs = 100, channels = 8, channel_gbs = 32, latency_ns = 80;
};

struct ScenarioConfig {
  std::string scenario = "msg";
  std::string topology = "torus";
  int nodes = 2;
  uint64_t bytes = 400;
  int repeat = 1;
  NetParams net;
  NicParams nic;
  MemoryParams memory;
  HostParams host;
  MpiParams mpi;
};

struct ScenarioResult {
  bool ok = false;
  std::string error;
  Time sim_time = 0;          // simulated time of the measured part
  uint64_t packets = 0;       // packets that crossed the network
  uint64_t events = 0;
  std::map<std::string, double> values;  // scenario-specific numbers (bandwidth, message counts ...)
  std::vector<std::string> lines;        // what the host programs printed
};

ScenarioResult run_scenario(const ScenarioConfig& cfg);

// Host programs written against the RDMA library / the message-passing layer (apps.cc):
// rdma-hello, rdma-msg, rdma-write, rdma-incast, rdma-incast-v2, rdma-barrier, rdma-sendrecv,
// rdma-test, imb.  run_scenario dispatches to them by name.
bool is_program(const std::string& scenario);
ScenarioResult run_program(const ScenarioConfig& cfg);

}  // namespace netsim
