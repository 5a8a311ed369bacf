// netsim: host programs on the RDMA library and the message-passing layer.
//
// The reference ships its NIC tests as C programs for the simulated nodes (tests/app/rdma/
// hello.c, msg.c, write.c, incast.c, incast-v2.c, barrier.c, sendrecv.c, test.c) and runs the
// Intel MPI Benchmarks over its MPI channel (tests/app/mpi).  The same programs are coroutines
// here: one per node, written against host.h / mpi.h, validating the data they move.
#include <algorithm>
#include <cinttypes>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <numeric>
#include <stdexcept>

#include "mpi.h"
#include "scenarios.h"

namespace netsim {

namespace {

using abi::Addr;

struct Ctx {
  const ScenarioConfig& cfg;
  Simulator sim;
  std::unique_ptr<Network> net;
  std::vector<std::unique_ptr<Nic>> nics;
  std::vector<std::unique_ptr<RdmaHost>> hosts;
  std::vector<std::unique_ptr<MiniMpi>> mpis;
  ScenarioResult res;
  std::vector<std::string> failures;
  std::vector<double> scratch;   // per-rank numbers that a real job would gather with a collective
  ProcSet procs;                 // last member: destroyed first, while everything it uses is alive
  explicit Ctx(const ScenarioConfig& c) : cfg(c) {
    net = make_network(sim, c.topology, c.nodes, c.net);
    for (int i = 0; i < c.nodes; ++i) {
      nics.push_back(std::make_unique<Nic>(sim, *net, i, c.nic));
      hosts.push_back(std::make_unique<RdmaHost>(*nics.back(), c.host));
      mpis.push_back(std::make_unique<MiniMpi>(*hosts.back(), c.mpi));
    }
    scratch.assign(c.nodes, 0.0);
  }
  int n() const { return cfg.nodes; }
  void say(const std::string& s) { res.lines.push_back(s); }
  void check(bool ok, const std::string& what) {
    if (!ok) failures.push_back(what);
  }
};

std::string fmt(const char* f, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, f);
  std::vsnprintf(buf, sizeof buf, f, ap);
  va_end(ap);
  return buf;
}

void fill(RdmaHost& h, Addr a, uint32_t len, int seed) {
  uint8_t* p = h.mem().ptr(a, len);
  for (uint32_t i = 0; i < len; ++i) p[i] = (uint8_t)((i * 7 + seed) & 0xff);
}
bool filled(RdmaHost& h, Addr a, uint32_t len, int seed) {
  const uint8_t* p = h.mem().ptr(a, len);
  for (uint32_t i = 0; i < len; ++i)
    if (p[i] != (uint8_t)((i * 7 + seed) & 0xff)) return false;
  return true;
}

// ---- hello: bring the library up and down -----------------------------------------------------
Co<void> hello(Ctx& c, int me) {
  RdmaHost& h = *c.hosts[me];
  c.check(co_await h.init() == 0, "init");
  co_await h.barrier();
  if (me == 0) c.say(fmt("hello: %d nodes are up", h.num_nodes()));
  c.check(co_await h.fini() == 0, "fini");
}

// ---- msg: node 0 sends cfg.bytes to node 1, which validates them --------------------------------
Co<void> msg(Ctx& c, int me) {
  RdmaHost& h = *c.hosts[me];
  const uint32_t len = (uint32_t)c.cfg.bytes;
  co_await h.init();
  const int cq = co_await h.create_cq();
  const int rq = co_await h.create_rq(0xbeef, cq);
  const Addr buf = h.mem().alloc(len);
  if (me == 1) co_await h.recv_post(buf, len, rq, 0x12345678);
  co_await h.barrier();   // the receive is posted before the sender starts
  if (me == 0) {
    fill(h, buf, len, 3);
    const Time t0 = c.sim.now();
    c.check(co_await h.send_post(buf, len, 1, 0xbeef, cq, 0xf00dbeef) == 0, "send_post");
    const auto e = co_await h.read_comp(cq);
    c.check(e.context == 0xf00dbeef, "send completion context");
    c.res.values["send_us"] = (c.sim.now() - t0) / 1e6;
  } else if (me == 1) {
    const auto e = co_await h.read_comp(cq);
    c.check(e.context == 0x12345678 && e.length == len && e.src_node == 0, "receive completion fields");
    c.check(filled(h, buf, len, 3), "payload");
    c.res.sim_time = c.sim.now();
    c.say(fmt("msg: node 1 received %u bytes from node %d, data ok", e.length, e.src_node));
  }
  co_await h.barrier();
  co_await h.fini();
}

// ---- write: one-sided write into node 1's region, then read it back ----------------------------
Co<void> write_read(Ctx& c, int me) {
  RdmaHost& h = *c.hosts[me];
  const uint32_t len = (uint32_t)c.cfg.bytes;
  co_await h.init();
  const int cq = co_await h.create_cq();
  Addr region = 0;
  if (me == 1) {
    region = h.mem().alloc(len + 64);
    c.check(co_await h.memory_reg(0x1234, region, len + 64) == 0, "memory_reg");
  }
  co_await h.barrier();
  if (me == 0) {
    const Addr src = h.mem().alloc(len), back = h.mem().alloc(len);
    fill(h, src, len, 9);
    c.check(co_await h.memory_write(0x1234, 1, 64, src, len, cq, 1) == 0, "memory_write");
    c.check((co_await h.read_comp(cq)).context == 1, "write completion");
    c.check(co_await h.memory_read(0x1234, 1, 64, back, len, cq, 2) == 0, "memory_read");
    const auto e = co_await h.read_comp(cq);
    c.check(e.context == 2 && e.length == len, "read completion");
    c.check(filled(h, back, len, 9), "read-back data");
    c.res.sim_time = c.sim.now();
    c.say(fmt("write: %u bytes written to node 1 and read back, data ok", len));
  }
  co_await h.barrier();
  if (me == 1) {
    c.check(filled(h, region + 64, len, 9), "region content on the target");
    co_await h.memory_unreg(0x1234);
  }
  co_await h.fini();
}

// ---- incast: every node but 0 sends to node 0 --------------------------------------------------
Co<void> incast(Ctx& c, int me) {
  RdmaHost& h = *c.hosts[me];
  const uint32_t len = (uint32_t)c.cfg.bytes;
  const int n = c.n();
  co_await h.init();
  const int cq = co_await h.create_cq();
  const int rq = co_await h.create_rq(0xbeef, cq);
  std::vector<Addr> bufs;
  if (me == 0)
    for (int i = 1; i < n; ++i) {
      bufs.push_back(h.mem().alloc(len));
      co_await h.recv_post(bufs.back(), len, rq, (uint64_t)i);
    }
  co_await h.barrier();
  const Time t0 = c.sim.now();
  if (me == 0) {
    std::vector<int> seen(n, 0);
    for (int i = 1; i < n; ++i) {
      const auto e = co_await h.read_comp(cq);
      c.check(e.src_node >= 1 && e.src_node < n && !seen[e.src_node], "one message per sender");
      if (e.src_node >= 1 && e.src_node < n) seen[e.src_node] = 1;
      c.check(filled(h, bufs[e.context - 1], len, e.src_node), "payload of an incast message");
    }
    c.res.sim_time = c.sim.now() - t0;
    c.res.values["ingress_gb_per_s"] = (double)len * (n - 1) / ((c.sim.now() - t0) * 1e-12) / 1e9;
    c.say(fmt("incast: node 0 received %d messages of %u bytes", n - 1, len));
  } else {
    const Addr src = h.mem().alloc(len);
    fill(h, src, len, me);
    co_await h.send_post(src, len, 0, 0xbeef, cq, 7);
    co_await h.read_comp(cq);
  }
  co_await h.barrier();
  co_await h.fini();
}

// ---- incast-v2: one-sided writes into per-sender slots of node 0, then a short notification -----
Co<void> incast_v2(Ctx& c, int me) {
  RdmaHost& h = *c.hosts[me];
  const uint32_t len = (uint32_t)c.cfg.bytes;
  const int n = c.n();
  co_await h.init();
  const int cq = co_await h.create_cq();
  const int rq = co_await h.create_rq(0xcafe, cq);
  Addr region = 0, notes = 0;
  if (me == 0) {
    region = h.mem().alloc((uint64_t)len * (n - 1));
    notes = h.mem().alloc(64 * (uint64_t)(n - 1));
    co_await h.memory_reg(0x77, region, (uint64_t)len * (n - 1));
    for (int i = 1; i < n; ++i) co_await h.recv_post(notes + 64 * (uint64_t)(i - 1), 64, rq, (uint64_t)i);
  }
  co_await h.barrier();
  const Time t0 = c.sim.now();
  if (me == 0) {
    for (int i = 1; i < n; ++i) co_await h.read_comp(cq);
    for (int i = 1; i < n; ++i) c.check(filled(h, region + (uint64_t)(i - 1) * len, len, i), "slot of a sender");
    c.res.sim_time = c.sim.now() - t0;
    c.say(fmt("incast-v2: %d slots of %u bytes written into node 0", n - 1, len));
  } else {
    const Addr src = h.mem().alloc(len), note = h.mem().alloc(64);
    fill(h, src, len, me);
    co_await h.memory_write(0x77, 0, (uint64_t)(me - 1) * len, src, len, cq, 1);
    co_await h.read_comp(cq);
    // the notification travels behind the data on the same virtual channel
    co_await h.send_post(note, 4, 0, 0xcafe, cq, 2);
    co_await h.read_comp(cq);
  }
  co_await h.barrier();
  co_await h.fini();
}

// ---- barrier ---------------------------------------------------------------------------------
Co<void> barrier_prog(Ctx& c, int me) {
  RdmaHost& h = *c.hosts[me];
  co_await h.init();
  co_await h.barrier();
  const Time t0 = c.sim.now();
  for (int i = 0; i < c.cfg.repeat; ++i) co_await h.barrier();
  if (me == 0) {
    c.res.sim_time = c.sim.now() - t0;
    c.res.values["us_per_barrier"] = (c.sim.now() - t0) / 1e6 / c.cfg.repeat;
    c.say(fmt("barrier: %d rounds on %d nodes", c.cfg.repeat, c.n()));
  }
  co_await h.fini();
}

// ---- sendrecv: ring exchange of cfg.bytes (phantom memory above 1 MiB) ---------------------------
Co<void> sendrecv(Ctx& c, int me) {
  RdmaHost& h = *c.hosts[me];
  const uint32_t len = (uint32_t)c.cfg.bytes;
  const int n = c.n();
  const bool phantom = len > (1u << 20);
  co_await h.init();
  const int cq = co_await h.create_cq();
  const int rq = co_await h.create_rq(0xbeef, cq);
  const Addr sbuf = h.mem().alloc(len, phantom), rbuf = h.mem().alloc(len, phantom);
  if (!phantom) fill(h, sbuf, len, me);
  co_await h.recv_post(rbuf, len, rq, 1);
  co_await h.barrier();
  const Time t0 = c.sim.now();
  co_await h.send_post(sbuf, len, (me + 1) % n, 0xbeef, cq, 2);
  co_await h.read_comp(cq);
  co_await h.read_comp(cq);   // the send's and the receive's completion, in either order
  c.scratch[me] = (double)(c.sim.now() - t0);
  if (!phantom) c.check(filled(h, rbuf, len, (me - 1 + n) % n), "ring payload");
  co_await h.barrier();
  if (me == 0) {
    const double worst = *std::max_element(c.scratch.begin(), c.scratch.end());
    c.res.sim_time = (Time)worst;
    c.res.values["exchange_us"] = worst / 1e6;
    c.res.values["gb_per_s_per_node"] = (double)len / (worst * 1e-12) / 1e9;
    c.say(fmt("sendrecv: ring exchange of %u bytes on %d nodes", len, n));
  }
  co_await h.fini();
}

// ---- test: the library's error paths and resource limits ----------------------------------------
Co<void> api_test(Ctx& c, int me) {
  RdmaHost& h = *c.hosts[me];
  co_await h.init();
  int checks = 0;
  auto expect = [&](bool ok, const char* what) {
    ++checks;
    c.check(ok, what);
  };
  if (me == 0) {
    std::vector<int> cqs;
    for (int i = 0; i < abi::kNumCompQ; ++i) cqs.push_back(co_await h.create_cq());
    expect(std::all_of(cqs.begin(), cqs.end(), [](int v) { return v >= 0; }), "sixteen completion queues");
    expect(co_await h.create_cq() == abi::kNoResources, "a seventeenth completion queue is refused");
    expect(co_await h.destroy_cq(cqs.back()) == 0, "destroy_cq");
    expect(co_await h.destroy_cq(cqs.back()) == abi::kBadId, "destroying twice is refused");
    const int rq = co_await h.create_rq(0x55, cqs[0]);
    expect(rq >= 0, "create_rq");
    expect(co_await h.destroy_cq(cqs[0]) == abi::kBadId, "a completion queue in use cannot be destroyed");
    expect(co_await h.create_rq(0x56, 1234) == abi::kBadId, "create_rq on an unknown completion queue");
    expect(co_await h.destroy_rq(rq) == 0, "destroy_rq");
    expect(co_await h.destroy_cq(cqs[0]) == 0, "destroy_cq after its receive queue is gone");
    const Addr buf = h.mem().alloc(256);
    expect(co_await h.send_post(buf, 512, 1, 0x55, cqs[1], 0) == abi::kBadAddress, "send beyond the allocation");
    expect(co_await h.send_post(buf, 16, 99, 0x55, cqs[1], 0) == abi::kBadId, "send to an unknown node");
    expect(co_await h.send_post(buf, 16, 1, 0x55, 1234, 0) == abi::kBadId, "send with an unknown completion queue");
    expect(co_await h.memory_reg(7, buf + 128, 512) == abi::kBadAddress, "registering beyond the allocation");
    expect(co_await h.memory_reg(7, buf, 256) == 0, "memory_reg");
    expect(co_await h.memory_unreg(7) == 0, "memory_unreg");
    expect(!h.comp_ready(cqs[1]), "no completion without traffic");
    c.say(fmt("test: %d library checks", checks));
  }
  co_await h.barrier();
  co_await h.fini();
}

// ---- imb: the point-to-point and collective timing loops of the Intel MPI Benchmarks -------------
struct ImbRow {
  std::string bench;
  uint32_t bytes;
  double t_avg_us;
};

Co<void> imb(Ctx& c, int me) {
  MiniMpi& mpi = *c.mpis[me];
  RdmaHost& h = *c.hosts[me];
  const int n = c.n(), iters = std::max(1, c.cfg.repeat);
  co_await mpi.init();
  std::vector<uint32_t> sizes;
  for (uint32_t s = 1; s <= std::max<uint64_t>(1, c.cfg.bytes); s *= 8) sizes.push_back(s);
  const uint32_t maxb = std::max<uint32_t>(4, sizes.back());
  const Addr sbuf = h.mem().alloc((uint64_t)maxb * n), rbuf = h.mem().alloc((uint64_t)maxb * n);
  std::memset(h.mem().ptr(sbuf, (uint64_t)maxb * n), 1, (uint64_t)maxb * n);
  auto report = [&](const char* bench, uint32_t bytes, double my_us, bool pair_only) -> Co<void> {
    c.scratch[me] = my_us;
    co_await mpi.barrier();
    if (me == 0) {
      double sum = 0;
      const int cnt = pair_only ? 2 : n;
      for (int i = 0; i < cnt; ++i) sum += c.scratch[i];
      c.say(fmt("imb %-14s %8u bytes  t_avg %10.3f us", bench, bytes, sum / cnt));
      c.res.values[std::string(bench) + "_" + std::to_string(bytes) + "_us"] = sum / cnt;
    }
    co_await mpi.barrier();
  };
  for (uint32_t s : sizes) {   // PingPong: half the round trip between ranks 0 and 1
    co_await mpi.barrier();
    double t = 0;
    if (me < 2) {
      const double t0 = mpi.wtime();
      for (int i = 0; i < iters; ++i) {
        if (me == 0) {
          co_await mpi.send(sbuf, s, 1, 1);
          co_await mpi.recv(rbuf, s, 1, 1);
        } else {
          co_await mpi.recv(rbuf, s, 0, 1);
          co_await mpi.send(sbuf, s, 0, 1);
        }
      }
      t = (mpi.wtime() - t0) / iters / 2 * 1e6;
    }
    co_await report("PingPong", s, t, true);
  }
  for (uint32_t s : sizes) {   // PingPing: both ranks send at once
    co_await mpi.barrier();
    double t = 0;
    if (me < 2) {
      const double t0 = mpi.wtime();
      for (int i = 0; i < iters; ++i) co_await mpi.sendrecv(sbuf, s, 1 - me, 2, rbuf, s, 1 - me, 2);
      t = (mpi.wtime() - t0) / iters * 1e6;
    }
    co_await report("PingPing", s, t, true);
  }
  for (uint32_t s : sizes) {   // Sendrecv: periodic chain
    co_await mpi.barrier();
    const double t0 = mpi.wtime();
    for (int i = 0; i < iters; ++i) co_await mpi.sendrecv(sbuf, s, (me + 1) % n, 3, rbuf, s, (me - 1 + n) % n, 3);
    co_await report("Sendrecv", s, (mpi.wtime() - t0) / iters * 1e6, false);
  }
  for (uint32_t s : sizes) {
    const uint32_t count = std::max<uint32_t>(1, s / 4);
    co_await mpi.barrier();
    double t0 = mpi.wtime();
    for (int i = 0; i < iters; ++i) co_await mpi.allreduce(sbuf, rbuf, count);
    co_await report("Allreduce", count * 4, (mpi.wtime() - t0) / iters * 1e6, false);
    c.check(h.mem().load<int32_t>(rbuf) == 0x01010101 * n, "allreduce sum");
    co_await mpi.barrier();
    t0 = mpi.wtime();
    for (int i = 0; i < iters; ++i) co_await mpi.reduce_scatter(sbuf, rbuf, count);
    co_await report("Reduce_scatter", count * 4, (mpi.wtime() - t0) / iters * 1e6, false);
    c.check(h.mem().load<int32_t>(rbuf) == 0x01010101 * n, "reduce_scatter sum");
  }
  for (uint32_t s : sizes) {
    co_await mpi.barrier();
    double t0 = mpi.wtime();
    for (int i = 0; i < iters; ++i) co_await mpi.allgather(sbuf, s, rbuf);
    co_await report("Allgather", s, (mpi.wtime() - t0) / iters * 1e6, false);
    co_await mpi.barrier();
    t0 = mpi.wtime();
    for (int i = 0; i < iters; ++i) co_await mpi.alltoall(sbuf, s, rbuf);
    co_await report("Alltoall", s, (mpi.wtime() - t0) / iters * 1e6, false);
    co_await mpi.barrier();
    t0 = mpi.wtime();
    for (int i = 0; i < iters; ++i) co_await mpi.bcast(sbuf, s, i % n);
    co_await report("Bcast", s, (mpi.wtime() - t0) / iters * 1e6, false);
  }
  {
    co_await mpi.barrier();
    const double t0 = mpi.wtime();
    for (int i = 0; i < iters; ++i) co_await mpi.barrier();
    co_await report("Barrier", 0, (mpi.wtime() - t0) / iters * 1e6, false);
  }
  if (me == 0) {
    c.res.sim_time = c.sim.now();
    c.res.values["eager_sent"] = (double)mpi.stats().eager_sent;
    c.res.values["rendezvous_sent"] = (double)mpi.stats().rndv_sent;
    c.res.values["credit_msgs"] = (double)mpi.stats().credit_msgs;
  }
  co_await mpi.finalize();
}

using Program = Co<void> (*)(Ctx&, int);

Program find_program(const std::string& name) {
  if (name == "rdma-hello") return hello;
  if (name == "rdma-msg") return msg;
  if (name == "rdma-write") return write_read;
  if (name == "rdma-incast") return incast;
  if (name == "rdma-incast-v2") return incast_v2;
  if (name == "rdma-barrier") return barrier_prog;
  if (name == "rdma-sendrecv") return sendrecv;
  if (name == "rdma-test") return api_test;
  if (name == "imb") return imb;
  return nullptr;
}

}  // namespace

bool is_program(const std::string& scenario) { return find_program(scenario) != nullptr; }

ScenarioResult run_program(const ScenarioConfig& cfg) {
  Program prog = find_program(cfg.scenario);
  if (!prog) throw std::invalid_argument("unknown program '" + cfg.scenario + "'");
  if (cfg.nodes < 2) throw std::invalid_argument("programs need at least two nodes");
  Ctx c(cfg);
  for (int i = 0; i < cfg.nodes; ++i) c.procs.spawn(prog(c, i));
  const bool drained = c.sim.run();
  ScenarioResult r = std::move(c.res);
  r.events = c.sim.events();
  r.packets = c.net->total_packets();
  if (r.sim_time == 0) r.sim_time = c.sim.now();
  if (!drained) r.error = "event limit reached";
  for (auto& n : c.nics)
    if (!n->last_error.empty() && r.error.empty()) r.error = n->last_error;
  for (auto& e : c.procs.errors())
    if (r.error.empty()) r.error = e;
  if (r.error.empty() && c.procs.finished() != c.procs.started())
    r.error = "deadlock: " + std::to_string(c.procs.started() - c.procs.finished()) + " of " +
              std::to_string(c.procs.started()) + " programs still waiting";
  if (r.error.empty() && !c.failures.empty()) r.error = "check failed: " + c.failures.front();
  uint64_t cmds = 0, ring_full = 0;
  for (auto& h : c.hosts) {
    cmds += h->stats().commands;
    ring_full += h->stats().ring_full_waits;
  }
  r.values["commands"] = (double)cmds;
  r.values["ring_full_waits"] = (double)ring_full;
  r.ok = r.error.empty();
  return r;
}

}  // namespace netsim
