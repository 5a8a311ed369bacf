// netsim unit tests (plain asserts; built with -fsanitize=address,undefined by the test driver).
#include <cassert>
#include <cstdio>

#include "scenarios.h"

using namespace netsim;

#define CHECK(c) do { if (!(c)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #c); return 1; } } while (0)

static int test_packetisation() {
  CHECK(packets_for(0) == 1);
  CHECK(packets_for(400) == 1);
  CHECK(packets_for(kMtu - kStreamHdrBytes) == 1);
  CHECK(packets_for(kMtu - kStreamHdrBytes + 1) == 2);
  CHECK(packets_for(10000) == (kStreamHdrBytes + 10000 + kMtu - 1) / kMtu);
  for (uint64_t len : {400ull, 5000ull, 100000ull}) {
    ScenarioConfig c;
    c.scenario = "msg";
    c.bytes = len;
    ScenarioResult r = run_scenario(c);
    CHECK(r.ok);
    CHECK(r.packets == packets_for((uint32_t)len));      // data packets only: no barrier in msg
    CHECK(r.values["data_ok"] == 1 && r.values["recv_length"] == (double)len);
  }
  return 0;
}

static int test_tree() {
  for (int n : {2, 5, 16, 21}) {
    int edges = 0;
    for (int i = 0; i < n; ++i) {
      Tree t(i, n, 4);
      CHECK((i == 0) == (t.parent < 0));
      for (int ch : t.children) {
        Tree c(ch, n, 4);
        CHECK(c.parent == i);
        ++edges;
      }
      CHECK(t.children.size() <= 4);
    }
    CHECK(edges == n - 1);
  }
  return 0;
}

static int test_barrier_counts() {
  for (int n : {2, 4, 8, 16}) {
    for (const char* topo : {"torus", "crossbar"}) {
      ScenarioConfig c;
      c.scenario = "barrier";
      c.nodes = n;
      c.topology = topo;
      c.repeat = 3;
      ScenarioResult r = run_scenario(c);
      CHECK(r.ok);
      CHECK(r.values["barrier_msgs"] == 2.0 * (n - 1) * 3);
    }
  }
  return 0;
}

static int test_mem_queue_fence_and_limit() {
  Simulator sim;
  NicParams p;
  p.max_mem_reqs = 4;
  MemRequestQ q(sim, p);
  q.record_order = true;
  std::vector<int> done;
  for (int i = 0; i < 6; ++i) q.request(2, 64, true, [&, i]() { done.push_back(i); });
  q.fence(2);
  q.request(2, 64, true, [&]() { done.push_back(100); });
  q.request(0, 16, true, [&]() { done.push_back(200); });
  sim.run();
  CHECK(q.max_pending_seen() <= 4);
  CHECK(done.size() == 8);
  // the request behind the fence completes after all six before it
  size_t pos100 = 0;
  for (size_t i = 0; i < done.size(); ++i) if (done[i] == 100) pos100 = i;
  for (size_t i = 0; i < done.size(); ++i) if (done[i] < 6) CHECK(i < pos100);
  // channel 0 was not blocked by the fence on channel 2
  size_t pos200 = 0;
  for (size_t i = 0; i < done.size(); ++i) if (done[i] == 200) pos200 = i;
  CHECK(pos200 < pos100);
  // round-robin: channel 0's request was issued before channel 2 drained
  CHECK(q.issued() == 8);
  return 0;
}

static int test_routing() {
  Simulator sim;
  NetParams p;
  Torus t(sim, {4, 4}, p);
  CHECK(t.hops(0, 0) == 2);            // up + down
  CHECK(t.hops(0, 1) == 3);
  CHECK(t.hops(0, 3) == 3);            // wrap-around
  CHECK(t.hops(0, 2) == 4);
  CHECK(t.hops(0, 10) == 6);           // (2,2): two hops per dimension
  Crossbar x(sim, 8, p);
  for (int d = 1; d < 8; ++d) CHECK(x.hops(0, d) == 2);
  return 0;
}

static int test_scenarios() {
  for (const char* s : {"write", "incast", "sendrecv", "allgather-ring", "allgather-direct"}) {
    for (const char* topo : {"torus", "crossbar"}) {
      ScenarioConfig c;
      c.scenario = s;
      c.topology = topo;
      c.nodes = 4;
      c.bytes = 20000;
      ScenarioResult r = run_scenario(c);
      if (!r.ok) std::printf("scenario %s/%s: %s\n", s, topo, r.error.c_str());
      CHECK(r.ok);
    }
  }
  // bandwidth is bounded by the slower of NIC link and memory path
  ScenarioConfig c;
  c.scenario = "sendrecv";
  c.nodes = 4;
  c.bytes = 4 << 20;
  ScenarioResult r = run_scenario(c);
  CHECK(r.ok);
  CHECK(r.values["gb_per_s_per_node"] > 1.0 && r.values["gb_per_s_per_node"] <= 16.0);
  // on a crossbar a direct all-gather beats the ring for small shards (one hop instead of n-1)
  ScenarioConfig a;
  a.nodes = 8;
  a.topology = "crossbar";
  a.bytes = 4096;
  a.scenario = "allgather-ring";
  const double ring = run_scenario(a).values["collective_us"];
  a.scenario = "allgather-direct";
  const double direct = run_scenario(a).values["collective_us"];
  CHECK(direct < ring);
  // a message without a posted receive is reported, not silently dropped
  {
    Simulator sim;
    NetParams np;
    NicParams nicp;
    auto net = make_network(sim, "crossbar", 2, np);
    Nic n0(sim, *net, 0, nicp), n1(sim, *net, 1, nicp);
    const int cq = n0.create_cq();
    n0.send_post(nullptr, 100, 1, 0xdead, cq, 1);
    sim.run();
    CHECK(!n1.last_error.empty());
  }
  return 0;
}

int main() {
  int rc = 0;
  rc |= test_packetisation();
  rc |= test_tree();
  rc |= test_barrier_counts();
  rc |= test_mem_queue_fence_and_limit();
  rc |= test_routing();
  rc |= test_scenarios();
  std::printf(rc == 0 ? "netsim tests passed\n" : "netsim tests FAILED\n");
  return rc;
}
