// netsim unit tests (plain asserts; built with -fsanitize=address,undefined by the test driver).
#include <cassert>
#include <cstdio>

#include <cstring>

#include "config.h"

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


// ---- host library, message passing, configuration ------------------------------------------------
static int test_abi_and_host_memory() {
  static_assert(sizeof(abi::NicCmd) == 64 && alignof(abi::NicCmd) == 64);
  static_assert(sizeof(abi::RdmaCompletion) == 16 && sizeof(abi::NicResp) == 16);
  HostMemory m;
  const abi::Addr a = m.alloc(100), b = m.alloc(64), ph = m.alloc(1 << 20, true);
  CHECK(a != b && m.bytes_allocated() == 100 + 64 + (1 << 20));
  m.store<uint32_t>(a + 96, 0xdeadbeef);
  CHECK(m.load<uint32_t>(a + 96) == 0xdeadbeef);
  auto [buf, off] = m.translate(a + 10, 90);
  CHECK(buf && off == 10);
  CHECK(m.translate(ph + 5, 100).first == nullptr);
  bool threw = false;
  try { m.translate(a + 10, 91); } catch (const std::out_of_range&) { threw = true; }
  CHECK(threw);
  threw = false;
  try { m.translate(a + 4096, 1); } catch (const std::out_of_range&) { threw = true; }   // the guard page
  CHECK(threw);
  threw = false;
  try { m.ptr(ph, 4); } catch (const std::out_of_range&) { threw = true; }
  CHECK(threw);
  m.release(b);
  threw = false;
  try { m.translate(b, 1); } catch (const std::out_of_range&) { threw = true; }
  CHECK(threw);
  return 0;
}

static int test_host_programs() {
  for (const char* prog : {"rdma-hello", "rdma-msg", "rdma-write", "rdma-incast", "rdma-incast-v2", "rdma-barrier",
                           "rdma-sendrecv", "rdma-test"}) {
    for (const char* topo : {"torus", "crossbar"}) {
      ScenarioConfig c;
      c.scenario = prog;
      c.nodes = 5;
      c.topology = topo;
      c.bytes = 3000;   // three packets per message
      c.repeat = 2;
      ScenarioResult r = run_scenario(c);
      if (!r.ok) std::printf("%s on %s: %s\n", prog, topo, r.error.c_str());
      CHECK(r.ok);
      CHECK(!r.lines.empty());
    }
  }
  // a command ring of two slots and several programs issuing commands on one host: the library
  // has to wait for ring space, and every command still gets its own answer
  {
    Simulator sim;
    NetParams np;
    NicParams nicp;
    nicp.cmd_q_size = 2;
    auto net = make_network(sim, "crossbar", 2, np);
    Nic n0(sim, *net, 0, nicp), n1(sim, *net, 1, nicp);
    RdmaHost h0(n0), h1(n1);
    ProcSet procs;
    int rq = -1, posted = 0;
    auto setup = [&rq](RdmaHost& h) -> Co<void> {
      co_await h.init();
      const int cq = co_await h.create_cq();
      rq = co_await h.create_rq(0x9, cq);
    };
    procs.spawn(setup(h0));
    sim.run();
    CHECK(rq >= 0);
    auto worker = [&rq, &posted](RdmaHost& h) -> Co<void> {
      const abi::Addr b = h.mem().alloc(64);
      for (int i = 0; i < 5; ++i) posted += co_await h.recv_post(b, 64, rq, i) == 0;
    };
    for (int k = 0; k < 6; ++k) procs.spawn(worker(h0));
    sim.run();
    CHECK(procs.finished() == 7 && posted == 30);
    CHECK(h0.stats().ring_full_waits > 0 && h0.stats().commands == 2 + 30);
  }
  // completions beyond the ring's capacity are an error, not silent loss: 40 receives, nobody polls
  {
    Simulator sim;
    NetParams np;
    NicParams nicp;
    auto net = make_network(sim, "crossbar", 2, np);
    Nic n0(sim, *net, 0, nicp), n1(sim, *net, 1, nicp);
    RdmaHost h0(n0), h1(n1);
    ProcSet procs;
    auto sender = [](RdmaHost& h) -> Co<void> {
      co_await h.init();
      const int cq = co_await h.create_cq(64);
      const abi::Addr b = h.mem().alloc(64);
      co_await h.barrier();
      for (int i = 0; i < 40; ++i) co_await h.send_post(b, 8, 1, 0x1, cq, i);
    };
    auto receiver = [](RdmaHost& h) -> Co<void> {
      co_await h.init();
      const int cq = co_await h.create_cq();   // 32 entries
      const int rq = co_await h.create_rq(0x1, cq);
      const abi::Addr b = h.mem().alloc(64 * 40);
      for (int i = 0; i < 40; ++i) co_await h.recv_post(b + 64 * i, 64, rq, i);
      co_await h.barrier();
    };
    procs.spawn(sender(h0));
    procs.spawn(receiver(h1));
    sim.run();
    CHECK(procs.finished() == 2);
    CHECK(n1.last_error.find("overflow") != std::string::npos);
  }
  // a receive that nothing matches leaves its program suspended: reported as a deadlock
  {
    ScenarioConfig d;
    d.scenario = "rdma-msg";
    d.nodes = 2;
    d.bytes = 64;
    d.nic.barrier_degree = 4;
    Simulator sim;
    auto net = make_network(sim, "torus", 2, d.net);
    Nic n0(sim, *net, 0, d.nic), n1(sim, *net, 1, d.nic);
    RdmaHost h0(n0), h1(n1);
    ProcSet procs;
    auto waits = [](RdmaHost& h) -> Co<void> {
      co_await h.init();
      const int cq = co_await h.create_cq();
      co_await h.read_comp(cq);   // nothing will ever arrive
    };
    procs.spawn(waits(h0));
    sim.run();
    CHECK(procs.finished() == 0 && procs.started() == 1);   // and the frame is freed by ~ProcSet (ASan checks)
  }
  return 0;
}

static int test_message_passing() {
  // eager and rendezvous paths, several node counts (powers of two and not), both topologies
  for (int n : {2, 3, 4, 6, 8}) {
    ScenarioConfig c;
    c.scenario = "imb";
    c.nodes = n;
    c.topology = n == 6 ? "torus:3x2" : (n == 8 ? "torus:2x2x2" : "crossbar");
    c.bytes = 32768;       // 1, 8, 64, 512, 4096 eager; 32768 rendezvous
    c.repeat = 2;
    ScenarioResult r = run_scenario(c);
    if (!r.ok) std::printf("imb on %d nodes: %s\n", n, r.error.c_str());
    CHECK(r.ok);
    CHECK(r.values["rendezvous_sent"] > 0 && r.values["eager_sent"] > 0);
    CHECK(r.values["PingPong_1_us"] > 0 && r.values["PingPong_32768_us"] > r.values["PingPong_1_us"]);
    CHECK(r.values["Alltoall_4096_us"] >= r.values["Sendrecv_4096_us"] * 0.5);
  }
  // few pre-posted buffers: the credit scheme must keep an all-to-all from overrunning them
  ScenarioConfig c;
  c.scenario = "imb";
  c.nodes = 8;
  c.topology = "crossbar";
  c.bytes = 512;
  c.repeat = 6;
  c.mpi.posted_recvs = 28;   // four credits per peer, the minimum
  ScenarioResult r = run_scenario(c);
  if (!r.ok) std::printf("imb with 28 buffers: %s\n", r.error.c_str());
  CHECK(r.ok);
  CHECK(r.values["credit_msgs"] > 0);
  c.mpi.posted_recvs = 16;   // too few: refused with a message, not a stall
  r = run_scenario(c);
  CHECK(!r.ok && r.error.find("posted_recvs") != std::string::npos);
  // payload correctness of point-to-point and collectives with real data
  {
    Simulator sim;
    NetParams np;
    NicParams nicp;
    const int n = 5;
    auto net = make_network(sim, "crossbar", n, np);
    std::vector<std::unique_ptr<Nic>> nics;
    std::vector<std::unique_ptr<RdmaHost>> hosts;
    std::vector<std::unique_ptr<MiniMpi>> mpis;
    for (int i = 0; i < n; ++i) {
      nics.push_back(std::make_unique<Nic>(sim, *net, i, nicp));
      hosts.push_back(std::make_unique<RdmaHost>(*nics.back()));
      mpis.push_back(std::make_unique<MiniMpi>(*hosts.back()));
    }
    int bad = 0;
    int badv[8] = {0};
    ProcSet procs;
    auto prog = [&bad, &badv, n](MiniMpi& mpi) -> Co<void> {
      HostMemory& m = mpi.host().mem();
      const int me = mpi.rank();
      co_await mpi.init();
      const uint32_t count = 3000;   // 12000 bytes: rendezvous
      const abi::Addr s = m.alloc(count * 4 * n), r = m.alloc(count * 4 * n);
      auto* sp = reinterpret_cast<int32_t*>(m.ptr(s, count * 4 * n));
      auto* rp = reinterpret_cast<int32_t*>(m.ptr(r, count * 4 * n));
      for (uint32_t i = 0; i < count * n; ++i) sp[i] = (int32_t)(i + 1000 * me);
      co_await mpi.allreduce(s, r, count);
      for (uint32_t i = 0; i < count; ++i) bad += rp[i] != (int32_t)(n * i + 1000 * (n * (n - 1) / 2));
      badv[0] = bad;
      co_await mpi.reduce_scatter(s, r, count);
      for (uint32_t i = 0; i < count; ++i)
        bad += rp[i] != (int32_t)(n * (me * count + i) + 1000 * (n * (n - 1) / 2));
      badv[1] = bad;
      co_await mpi.allgather(s, 64, r);
      for (int k = 0; k < n; ++k) bad += rp[k * 16 + 3] != 3 + 1000 * k;
      badv[2] = bad;
      co_await mpi.alltoall(s, 64, r);
      for (int k = 0; k < n; ++k) bad += rp[k * 16 + 2] != (int32_t)(me * 16 + 2 + 1000 * k);
      badv[3] = bad;
      if (me == 2) sp[7] = 424242;
      co_await mpi.bcast(s, count * 4, 2);
      bad += sp[7] != 424242;
      badv[4] = bad;
      // unexpected messages: the sends arrive long before the receives are posted, tags out of order
      if (me == 0) {
        co_await mpi.send(s, 100, 1, 5);
        co_await mpi.send(s + 400, 100, 1, 6);
      } else if (me == 1) {
        co_await mpi.host().compute(50 * kUs);
        co_await mpi.recv(r, 100, 0, 6);
        co_await mpi.recv(r + 400, 100, MiniMpi::kAnySource, 5);
        // after the broadcast every rank's send buffer holds rank 2's values i + 2000
        bad += rp[0] != 2100 || rp[24] != 2124;           // tag 6 carried elements 100..124
        bad += rp[100] != 2000 || rp[107] != 424242;      // tag 5 carried elements 0..24
        bad += mpi.stats().unexpected < 1;                // tag 5 arrived first and had to wait
      }
      co_await mpi.finalize();
    };
    for (int i = 0; i < n; ++i) procs.spawn(prog(*mpis[i]));
    sim.run();
    for (auto& e : procs.errors()) std::printf("program error: %s\n", e.c_str());
    for (auto& nic : nics)
      if (!nic->last_error.empty()) std::printf("nic error: %s\n", nic->last_error.c_str());
    CHECK(procs.finished() == n && procs.errors().empty());
    if (bad) std::printf("bad after allreduce %d reduce_scatter %d allgather %d alltoall %d bcast %d total %d\n", badv[0], badv[1], badv[2], badv[3], badv[4], bad);
    CHECK(bad == 0);
  }
  return 0;
}

static int test_config_files() {
  ScenarioConfig c;
  std::string err;
  CHECK(apply_setting("network", "link_gbs", "900", c, err) && c.net.link_bw == 900e9);
  CHECK(apply_setting("memory", "kind", "hbm", c, err));
  CHECK(apply_setting("memory", "channels", "4", c, err) && apply_setting("memory", "channel_gbs", "50", c, err));
  CHECK(c.nic.mem_bw == 200e9);
  CHECK(!apply_setting("network", "link_gbz", "1", c, err) && err.find("unknown key") != std::string::npos);
  err.clear();
  CHECK(!apply_setting("nope", "x", "1", c, err) && err.find("unknown section") != std::string::npos);
  err.clear();
  CHECK(!apply_setting("nic", "cmd_q_size", "many", c, err) && err.find("not a number") != std::string::npos);
  err.clear();
  CHECK(!apply_setting("run", "nodes", "0", c, err));
  // a dumped configuration reads back to the same text
  const std::string text = dump_config(c);
  const char* path = "netsim_test_roundtrip.ini";
  {
    FILE* f = std::fopen(path, "w");
    CHECK(f != nullptr);
    std::fputs(text.c_str(), f);
    std::fclose(f);
  }
  ScenarioConfig d;
  err.clear();
  const bool ok = load_config(path, d, err);
  std::remove(path);
  if (!ok) std::printf("%s\n", err.c_str());
  CHECK(ok);
  CHECK(dump_config(d) == text);
  CHECK(!load_config("does_not_exist.ini", d, err));
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
  rc |= test_abi_and_host_memory();
  rc |= test_host_programs();
  rc |= test_message_passing();
  rc |= test_config_files();
  std::printf(rc == 0 ? "netsim tests passed\n" : "netsim tests FAILED\n");
  return rc;
}
