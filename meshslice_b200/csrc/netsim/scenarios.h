// netsim: scripted scenarios (the reference's RDMA test programs msg / write / incast / barrier /
// sendrecv, tests/app/rdma/*.c, as event-driven scripts) and simple collectives built on the
// one-sided API, used to produce latency / bandwidth curves comparable to a collectives sweep.
#pragma once
#include <map>
#include <string>

#include "nic.h"

namespace netsim {

struct ScenarioConfig {
  std::string scenario = "msg";
  std::string topology = "torus";
  int nodes = 2;
  uint64_t bytes = 400;
  int repeat = 1;
  NetParams net;
  NicParams nic;
};

struct ScenarioResult {
  bool ok = false;
  std::string error;
  Time sim_time = 0;          // simulated time of the measured part
  uint64_t packets = 0;       // packets that crossed the network
  uint64_t events = 0;
  std::map<std::string, double> values;  // scenario-specific numbers (bandwidth, message counts ...)
};

ScenarioResult run_scenario(const ScenarioConfig& cfg);

}  // namespace netsim
