// netsim: scenario scripts.  Every node is driven by completion callbacks; nothing blocks.
#include "scenarios.h"

#include <stdexcept>

namespace netsim {

namespace {

struct World {
  Simulator sim;
  std::unique_ptr<Network> net;
  std::vector<std::unique_ptr<Nic>> nics;
  explicit World(const ScenarioConfig& c) {
    net = make_network(sim, c.topology, c.nodes, c.net);
    for (int i = 0; i < c.nodes; ++i) nics.push_back(std::make_unique<Nic>(sim, *net, i, c.nic));
  }
  std::string first_error() const {
    for (auto& n : nics)
      if (!n->last_error.empty()) return n->last_error;
    return "";
  }
};

Buffer make_buf(uint64_t bytes, int fill = -1) {
  auto b = std::make_shared<std::vector<uint8_t>>(bytes);
  if (fill >= 0)
    for (uint64_t i = 0; i < bytes; ++i) (*b)[i] = static_cast<uint8_t>((i * 7 + fill) & 0xff);
  return b;
}

void finish(World& w, ScenarioResult& r) {
  const bool done = w.sim.run();
  r.events = w.sim.events();
  r.packets = w.net->total_packets();
  if (!done) r.error = "event limit reached";
  const std::string e = w.first_error();
  if (!e.empty()) r.error = e;
}

// node 0 sends `bytes` to node 1, which posted a receive; both wait for their completion
ScenarioResult msg(const ScenarioConfig& c) {
  ScenarioResult r;
  World w(c);
  const uint32_t len = (uint32_t)c.bytes;
  Buffer src = make_buf(len, 3), dst = make_buf(len);
  int got = 0;
  Time t_recv = 0;
  for (int n = 0; n < 2; ++n) {
    Nic& nic = *w.nics[n];
    const int cq = nic.create_cq();
    const int rq = nic.create_rq(0xbeef, cq);
    if (n == 0) {
      nic.send_post(src, len, 1, 0xbeef, cq, 0xf00dbeef);
      nic.on_completion(cq, [&](const Completion&) { ++got; });
    } else {
      nic.recv_post(dst, len, rq, 0x12345678);
      nic.on_completion(cq, [&](const Completion& comp) {
        ++got;
        t_recv = comp.time;
        r.values["recv_context_ok"] = comp.context == 0x12345678 ? 1 : 0;
        r.values["recv_length"] = comp.length;
      });
    }
  }
  finish(w, r);
  r.sim_time = t_recv;
  r.values["completions"] = got;
  r.values["data_ok"] = *src == *dst ? 1 : 0;
  r.values["packets_expected"] = packets_for(len);
  r.ok = r.error.empty() && got == 2 && *src == *dst;
  return r;
}

// node 1 registers a region; node 0 writes into it at an offset and reads it back
ScenarioResult write_read(const ScenarioConfig& c) {
  ScenarioResult r;
  World w(c);
  const uint32_t len = (uint32_t)c.bytes;
  Buffer region = make_buf(len + 64), data = make_buf(len, 9), back = make_buf(len);
  Nic &a = *w.nics[0], &b = *w.nics[1];
  const int cq = a.create_cq();
  b.memory_reg(0x1234, region);
  bool read_done = false;
  a.barrier([] {});
  b.barrier([&]() {});
  // the write has no remote completion; order it before the read with a barrier round
  a.memory_write(0x1234, 1, 64, data, len, cq, 1);
  a.on_completion(cq, [&](const Completion&) {
    a.memory_read(0x1234, 1, 64, back, len, cq, 2);
    a.on_completion(cq, [&](const Completion& comp) {
      read_done = comp.context == 2;
      r.sim_time = comp.time;
    });
  });
  finish(w, r);
  bool region_ok = true;
  for (uint32_t i = 0; i < len; ++i) region_ok &= (*region)[64 + i] == (*data)[i];
  r.values["region_ok"] = region_ok;
  r.values["readback_ok"] = *back == *data ? 1 : 0;
  r.ok = r.error.empty() && read_done && region_ok && *back == *data;
  return r;
}

// every node but 0 sends `bytes` to node 0
ScenarioResult incast(const ScenarioConfig& c) {
  ScenarioResult r;
  World w(c);
  const uint32_t len = (uint32_t)c.bytes;
  Nic& root = *w.nics[0];
  const int cq0 = root.create_cq();
  const int rq0 = root.create_rq(0xbeef, cq0);
  int received = 0;
  std::vector<Buffer> bufs;
  std::function<void()> wait_next = [&]() {
    root.on_completion(cq0, [&](const Completion& comp) {
      ++received;
      r.sim_time = comp.time;
      if (received < c.nodes - 1) wait_next();
    });
  };
  for (int i = 1; i < c.nodes; ++i) {
    bufs.push_back(make_buf(len));
    root.recv_post(bufs.back(), len, rq0, i);
  }
  wait_next();
  for (int i = 1; i < c.nodes; ++i) {
    Nic& n = *w.nics[i];
    const int cq = n.create_cq();
    n.barrier([] {});
    n.send_post(make_buf(len, i), len, 0, 0xbeef, cq, i);
  }
  root.barrier([] {});
  finish(w, r);
  r.values["received"] = received;
  r.ok = r.error.empty() && received == c.nodes - 1;
  return r;
}

ScenarioResult barrier(const ScenarioConfig& c) {
  ScenarioResult r;
  World w(c);
  int done = 0;
  std::vector<int> rounds(c.nodes, 0);
  std::function<void(int)> go = [&](int n) {
    w.nics[n]->barrier([&, n]() {
      ++done;
      r.sim_time = w.sim.now();
      if (++rounds[n] < c.repeat) go(n);
    });
  };
  for (int n = 0; n < c.nodes; ++n) go(n);
  finish(w, r);
  uint64_t msgs = 0;
  for (auto& n : w.nics) msgs += n->stats().barrier_msgs_sent;
  r.values["barrier_msgs"] = (double)msgs;
  r.values["barrier_msgs_expected"] = 2.0 * (c.nodes - 1) * c.repeat;
  r.values["us_per_barrier"] = r.sim_time / 1e6 / c.repeat;
  r.ok = r.error.empty() && done == c.nodes * c.repeat && msgs == (uint64_t)(2 * (c.nodes - 1) * c.repeat);
  return r;
}

// ring exchange after a barrier: every node sends `bytes` to (me + 1) % n (sendrecv.c)
ScenarioResult sendrecv(const ScenarioConfig& c) {
  ScenarioResult r;
  World w(c);
  const uint32_t len = (uint32_t)c.bytes;
  int recvd = 0;
  Time t0 = 0;
  bool materialize = c.bytes <= (1u << 20);
  for (int n = 0; n < c.nodes; ++n) {
    Nic& nic = *w.nics[n];
    const int msg_cq = nic.create_cq(), cq = nic.create_cq();
    const int rq = nic.create_rq(0xbeef, msg_cq);
    nic.recv_post(materialize ? make_buf(len) : nullptr, len, rq, n);
    nic.barrier([&, n, cq, len, materialize]() {
      t0 = std::max(t0, w.sim.now());
      w.nics[n]->send_post(materialize ? make_buf(len, n) : nullptr, len, (n + 1) % c.nodes, 0xbeef, cq, 0xf00d);
    });
    nic.on_completion(msg_cq, [&](const Completion& comp) {
      ++recvd;
      r.sim_time = std::max(r.sim_time, comp.time);
    });
  }
  finish(w, r);
  const Time dt = r.sim_time > t0 ? r.sim_time - t0 : 0;
  r.values["exchange_us"] = dt / 1e6;
  r.values["gb_per_s_per_node"] = dt ? (double)len / (dt * 1e-12) / 1e9 : 0;
  r.sim_time = dt;
  r.ok = r.error.empty() && recvd == c.nodes;
  return r;
}

// all-gather of `bytes` per node with one-sided writes: 'ring' forwards n-1 times to the next
// node, 'direct' writes the own shard to every peer at once
ScenarioResult allgather(const ScenarioConfig& c, bool ring) {
  ScenarioResult r;
  World w(c);
  const int n = c.nodes;
  const uint32_t len = (uint32_t)c.bytes;
  std::vector<int> cq(n), rq(n), steps(n, 0);
  Time t0 = 0;
  int finished = 0;
  for (int i = 0; i < n; ++i) {
    cq[i] = w.nics[i]->create_cq();
    rq[i] = w.nics[i]->create_rq(0xa11, cq[i]);
    for (int k = 0; k < n - 1; ++k) w.nics[i]->recv_post(nullptr, len, rq[i], k);
  }
  std::function<void(int)> wait_recv = [&](int i) {
    w.nics[i]->on_completion(cq[i], [&, i](const Completion& comp) {
      if (comp.context == 0xf00d) { wait_recv(i); return; }   // own send completion
      ++steps[i];
      if (ring && steps[i] < n - 1) w.nics[i]->send_post(nullptr, len, (i + 1) % n, 0xa11, cq[i], 0xf00d);
      if (steps[i] == n - 1) {
        ++finished;
        r.sim_time = std::max(r.sim_time, comp.time);
      } else {
        wait_recv(i);
      }
    });
  };
  for (int i = 0; i < n; ++i) {
    w.nics[i]->barrier([&, i]() {
      t0 = std::max(t0, w.sim.now());
      if (ring) {
        w.nics[i]->send_post(nullptr, len, (i + 1) % n, 0xa11, cq[i], 0xf00d);
      } else {
        for (int k = 1; k < n; ++k) w.nics[i]->send_post(nullptr, len, (i + k) % n, 0xa11, cq[i], 0xf00d);
      }
    });
    wait_recv(i);
  }
  finish(w, r);
  const Time dt = r.sim_time > t0 ? r.sim_time - t0 : 0;
  r.values["collective_us"] = dt / 1e6;
  r.values["ingress_gb_per_s"] = dt ? (double)len * (n - 1) / (dt * 1e-12) / 1e9 : 0;
  r.sim_time = dt;
  r.ok = r.error.empty() && finished == n;
  return r;
}

}  // namespace

ScenarioResult run_scenario(const ScenarioConfig& c) {
  if (c.nodes < 2) throw std::invalid_argument("scenarios need at least two nodes");
  if (is_program(c.scenario)) return run_program(c);
  if (c.scenario == "msg") return msg(c);
  if (c.scenario == "write") return write_read(c);
  if (c.scenario == "incast") return incast(c);
  if (c.scenario == "barrier") return barrier(c);
  if (c.scenario == "sendrecv") return sendrecv(c);
  if (c.scenario == "allgather-ring") return allgather(c, true);
  if (c.scenario == "allgather-direct") return allgather(c, false);
  throw std::invalid_argument("unknown scenario '" + c.scenario + "'");
}

}  // namespace netsim
