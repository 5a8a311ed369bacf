// netsim: implementation of the network and NIC models declared in sim.h / nic.h.
#include <algorithm>
#include <cassert>
#include <cstring>
#include <numeric>
#include <sstream>
#include <stdexcept>

#include "nic.h"

namespace netsim {

// =============================================================================================
// Network
// =============================================================================================
void Network::send(const Packet& pkt) {
  ++total_packets_;
  auto p = std::make_shared<Packet>(pkt);
  auto path = std::make_shared<std::vector<int>>(route(pkt.src, pkt.dst));
  hop(p, path, 0);
}

void Network::hop(std::shared_ptr<Packet> pkt, std::shared_ptr<std::vector<int>> path, size_t i) {
  if (i == path->size()) {
    if (sinks_[pkt->dst]) sinks_[pkt->dst](*pkt);
    return;
  }
  Link& l = links_[(*path)[i]];
  const uint32_t wire = ((pkt->payload + kPktOverhead + p_.flit_bytes - 1) / p_.flit_bytes) * p_.flit_bytes;
  const Time start = std::max(sim_.now(), l.free_at);
  const Time ser = bytes_time(wire, l.bw);
  l.free_at = start + ser;
  LinkStats& s = stats_[(*path)[i]];
  s.packets++;
  s.bytes += wire;
  s.busy += ser;
  sim_.at(start + ser + l.latency, [this, pkt, path, i]() { hop(pkt, path, i + 1); });
}

Torus::Torus(Simulator& sim, std::vector<int> shape, NetParams p)
    : Network(sim, std::accumulate(shape.begin(), shape.end(), 1, std::multiplies<int>()), p), shape_(shape) {
  nic_up_.resize(n_);
  nic_down_.resize(n_);
  for (int i = 0; i < n_; ++i) {
    nic_up_[i] = add_link(p.nic_bw, p.link_latency + p.router_latency);
    nic_down_[i] = add_link(p.nic_bw, p.link_latency);
  }
  plus_.assign(shape.size(), std::vector<int>(n_));
  minus_.assign(shape.size(), std::vector<int>(n_));
  for (size_t d = 0; d < shape.size(); ++d)
    for (int i = 0; i < n_; ++i) {
      plus_[d][i] = add_link(p.link_bw, p.link_latency + p.router_latency);
      minus_[d][i] = add_link(p.link_bw, p.link_latency + p.router_latency);
    }
}

std::string Torus::name() const {
  std::ostringstream o;
  o << "torus(";
  for (size_t i = 0; i < shape_.size(); ++i) o << (i ? "x" : "") << shape_[i];
  o << ")";
  return o.str();
}

std::vector<int> Torus::coords(int node) const {
  std::vector<int> c(shape_.size());
  for (size_t d = 0; d < shape_.size(); ++d) {
    c[d] = node % shape_[d];
    node /= shape_[d];
  }
  return c;
}

std::vector<int> Torus::route(int src, int dst) {
  std::vector<int> path{nic_up_[src]};
  std::vector<int> cur = coords(src), tgt = coords(dst);
  int node = src;
  int stride = 1;
  for (size_t d = 0; d < shape_.size(); ++d) {
    const int n = shape_[d];
    int fwd = (tgt[d] - cur[d] + n) % n;
    const bool plus = fwd <= n - fwd;
    int steps = plus ? fwd : n - fwd;
    while (steps-- > 0) {
      path.push_back(plus ? plus_[d][node] : minus_[d][node]);
      const int next = plus ? (cur[d] + 1) % n : (cur[d] + n - 1) % n;
      node += (next - cur[d]) * stride;
      cur[d] = next;
    }
    stride *= n;
  }
  path.push_back(nic_down_[dst]);
  return path;
}

Crossbar::Crossbar(Simulator& sim, int nodes, NetParams p) : Network(sim, nodes, p) {
  up_.resize(nodes);
  down_.resize(nodes);
  for (int i = 0; i < nodes; ++i) {
    up_[i] = add_link(p.link_bw, p.link_latency + p.router_latency);
    down_[i] = add_link(p.link_bw, p.link_latency);
  }
}

std::unique_ptr<Network> make_network(Simulator& sim, const std::string& spec, int nodes, NetParams p) {
  if (spec.rfind("torus", 0) == 0) {
    std::vector<int> shape;
    const size_t c = spec.find(':');
    if (c == std::string::npos) {
      shape = {nodes};
    } else {
      std::stringstream ss(spec.substr(c + 1));
      std::string tok;
      while (std::getline(ss, tok, 'x')) shape.push_back(std::stoi(tok));
    }
    int prod = 1;
    for (int s : shape) prod *= s;
    if (prod != nodes) throw std::invalid_argument("torus shape does not match the node count");
    return std::make_unique<Torus>(sim, shape, p);
  }
  if (spec == "crossbar") return std::make_unique<Crossbar>(sim, nodes, p);
  throw std::invalid_argument("unknown topology '" + spec + "' (torus[:AxBx..] | crossbar)");
}

// =============================================================================================
// MemRequestQ
// =============================================================================================
void MemRequestQ::request(int channel, uint32_t bytes, bool is_write, std::function<void()> done) {
  chan_[channel].q.push_back(Req{bytes, is_write, false, std::move(done)});
  pump();
}

void MemRequestQ::fence(int channel) {
  chan_[channel].q.push_back(Req{0, false, true, nullptr});
  pump();
}

void MemRequestQ::pump() {
  // round-robin over the channels while the global limit allows another request
  bool progress = true;
  while (progress) {
    progress = false;
    for (int k = 0; k < 3; ++k) {
      const int c = (rr_ + k) % 3;
      Chan& ch = chan_[c];
      if (ch.q.empty()) continue;
      if (ch.q.front().is_fence) {
        if (ch.inflight == 0) {   // everything before the fence has completed
          ch.q.pop_front();
          progress = true;
        }
        continue;
      }
      if (pending_ >= p_.max_mem_reqs) return;
      Req r = std::move(ch.q.front());
      ch.q.pop_front();
      ++pending_;
      ++ch.inflight;
      ++issued_;
      max_seen_ = std::max(max_seen_, pending_);
      if (record_order) issue_order.push_back(c);
      const Time start = std::max(sim_.now(), port_free_);
      port_free_ = start + bytes_time(std::max<uint32_t>(r.bytes, 8), p_.mem_bw);
      auto done = std::move(r.done);
      sim_.at(port_free_ + p_.mem_latency, [this, c, done]() {
        --pending_;
        --chan_[c].inflight;
        if (done) done();
        pump();
      });
      rr_ = (c + 1) % 3;
      progress = true;
      break;
    }
  }
}

// =============================================================================================
// Tree
// =============================================================================================
Tree::Tree(int node, int n, int degree) {
  if (node > 0) parent = (node - 1) / degree;
  for (int k = 1; k <= degree; ++k) {
    const int c = node * degree + k;
    if (c < n) children.push_back(c);
  }
}

// =============================================================================================
// Nic
// =============================================================================================
Nic::Nic(Simulator& sim, Network& net, int node, NicParams p)
    : sim_(sim), net_(net), node_(node), p_(p), memq_(sim, p_), tree_(node, net.nodes(), (int)p.barrier_degree),
      send_fifo_(p.num_vcs), active_(p.num_vcs), out_q_(p.num_vcs), out_busy_(p.num_vcs, false) {
  net_.attach(node, [this](const Packet& pkt) { on_packet(pkt); });
}

void Nic::submit(std::function<void()> cmd) {
  // the host writes a 64-byte command over MMIO; the NIC dequeues one command per clock
  ++stats_.commands;
  if (finished_) {
    last_error = "node " + std::to_string(node_) + ": command after fini";
    return;
  }
  if (direct_) {   // the command ring in front of this NIC already accounted for the MMIO write
    cmd();
    return;
  }
  const Time arrive = std::max(sim_.now() + p_.host_cmd_latency, cmd_free_);
  cmd_free_ = arrive + p_.clock;
  sim_.at(arrive, std::move(cmd));
}

int Nic::create_cq() {
  cqs_.emplace_back();
  return (int)cqs_.size() - 1;
}

int Nic::create_rq(uint32_t key, int cq) {
  rqs_.push_back(RecvQueue{key, cq, {}});
  return (int)rqs_.size() - 1;
}

bool Nic::destroy_cq(int cq) {
  if (cq < 0 || cq >= (int)cqs_.size() || !cqs_[cq].alive) return false;
  for (auto& q : rqs_)
    if (q.alive && q.cq == cq) return false;
  cqs_[cq].alive = false;
  cqs_[cq].entries.clear();
  cqs_[cq].waiters.clear();
  return true;
}

bool Nic::destroy_rq(int rq) {
  if (rq < 0 || rq >= (int)rqs_.size() || !rqs_[rq].alive) return false;
  rqs_[rq].alive = false;
  rqs_[rq].posted.clear();
  return true;
}

void Nic::fini() {
  submit([this]() { finished_ = true; });
}

void Nic::recv_post(Buffer buf, uint32_t len, int rq, uint64_t context, uint64_t buf_off) {
  submit([=, this]() {
    if (rq < 0 || rq >= (int)rqs_.size() || !rqs_[rq].alive) {
      last_error = "node " + std::to_string(node_) + ": receive posted to an unknown queue";
      return;
    }
    rqs_[rq].posted.push_back(PostedRecv{buf, len, context, buf_off});
  });
}

void Nic::send_post(Buffer buf, uint32_t len, int dst, uint32_t rq_key, int cq, uint64_t context,
                    uint64_t buf_off) {
  submit([=, this]() {
    SendEntry e;
    e.hdr.type = StreamType::Msg;
    e.hdr.length = len;
    e.hdr.key = rq_key;
    e.dst = dst; e.vc = 0; e.cq = cq; e.context = context; e.src = buf; e.src_off = buf_off; e.payload_len = len;
    start_send(std::move(e));
  });
}

void Nic::memory_reg(uint32_t key, Buffer buf, uint64_t buf_off, uint64_t len) {
  submit([=, this]() { regions_[key] = Region{buf, buf_off, len}; });
}

void Nic::memory_unreg(uint32_t key) {
  submit([=, this]() { regions_.erase(key); });
}

void Nic::memory_write(uint32_t key, int dst, uint64_t offset, Buffer data, uint32_t len, int cq, uint64_t context,
                       uint64_t data_off) {
  submit([=, this]() {
    SendEntry e;
    e.hdr.type = StreamType::Write;
    e.hdr.length = len;
    e.hdr.key = key;
    e.hdr.offset = offset;
    e.dst = dst; e.vc = 0; e.cq = cq; e.context = context; e.src = data; e.src_off = data_off; e.payload_len = len;
    start_send(std::move(e));
  });
}

void Nic::memory_read(uint32_t key, int dst, uint64_t offset, Buffer into, uint32_t len, int cq, uint64_t context,
                      uint64_t into_off) {
  submit([=, this]() {
    const uint32_t rk = next_resp_key_++;
    reads_[rk] = PendingRead{into, cq, context, into_off};
    SendEntry e;
    e.hdr.type = StreamType::ReadReq;
    e.hdr.length = 0;
    e.hdr.key = key;
    e.hdr.offset = offset;
    e.hdr.read_len = len;
    e.hdr.resp_key = rk;
    e.dst = dst; e.vc = 0; e.cq = -1; e.context = 0; e.payload_len = 0;
    start_send(std::move(e));
  });
}

void Nic::on_completion(int cq, std::function<void(const Completion&)> fn) {
  CompQueue& q = cqs_[cq];
  if (!q.entries.empty()) {
    Completion c = q.entries.front();
    q.entries.pop_front();
    sim_.after(p_.host_poll_latency, [fn, c]() { fn(c); });
  } else {
    q.waiters.push_back(std::move(fn));
  }
}

void Nic::complete(int cq, Completion c) {
  if (cq < 0) return;
  // the completion entry is written to host memory on channel 0, behind a fence on the DMA
  // channel so that the host never sees the entry before the payload
  memq_.fence(2);
  memq_.request(0, 16, true, [this, cq, c]() mutable {
    c.time = sim_.now();
    if (cq_sink_) {   // the entry lands in a completion ring in host memory
      cq_sink_(cq, c);
      return;
    }
    CompQueue& q = cqs_[cq];
    if (!q.alive) return;
    if (!q.waiters.empty()) {
      auto fn = std::move(q.waiters.front());
      q.waiters.pop_front();
      sim_.after(p_.host_poll_latency, [fn, c]() { fn(c); });
    } else {
      q.entries.push_back(c);
    }
  });
}

// ---- send path -------------------------------------------------------------------------------
void Nic::start_send(SendEntry e) {
  const int vc = e.vc;
  send_fifo_[vc].push_back(std::move(e));
  pump_send(vc);
}

void Nic::pump_send(int vc) {
  ActiveSend& a = active_[vc];
  if (!a.active) {
    if (send_fifo_[vc].empty()) return;
    a = ActiveSend{};
    a.e = std::move(send_fifo_[vc].front());
    send_fifo_[vc].pop_front();
    a.stream_id = next_stream_++;
    a.seq_len = packets_for(a.e.payload_len);
    a.active = true;
    ++stats_.streams_sent;
  }
  // DMA-read the payload in 64-byte requests, at most send_ready_depth packets ahead
  const uint64_t total = a.e.payload_len;
  while (a.read_issued < total) {
    const uint64_t ahead_pkts = (a.read_issued + kStreamHdrBytes) / kMtu;
    if (ahead_pkts >= a.next_pkt + p_.send_ready_depth) break;
    const uint32_t n = (uint32_t)std::min<uint64_t>(p_.mem_req_bytes, total - a.read_issued);
    a.read_issued += n;
    memq_.request(2, n, false, [this, vc, n]() {
      active_[vc].read_done += n;
      emit_packets(vc);
    });
  }
  if (total == 0) emit_packets(vc);
}

void Nic::emit_packets(int vc) {
  ActiveSend& a = active_[vc];
  if (!a.active) return;
  while (a.next_pkt < a.seq_len) {
    // bytes of payload needed up to the end of packet next_pkt
    const uint64_t end = std::min<uint64_t>((uint64_t)(a.next_pkt + 1) * kMtu - kStreamHdrBytes, a.e.payload_len);
    if (a.read_done < end) break;
    if (out_q_[vc].size() >= p_.out_q_depth) break;   // back-pressure from the network queue
    const uint64_t begin = a.next_pkt == 0 ? 0 : (uint64_t)a.next_pkt * kMtu - kStreamHdrBytes;
    Packet p;
    p.kind = Packet::Stream;
    p.src = node_; p.dst = a.e.dst; p.vc = vc;
    p.stream_id = a.stream_id;
    p.seq = a.next_pkt; p.seq_len = a.seq_len;
    p.first = a.next_pkt == 0;
    p.payload = (uint32_t)(end - begin) + (p.first ? kStreamHdrBytes : 0);
    if (p.first) p.hdr = a.e.hdr;
    if (a.e.src && end > begin) {
      const uint64_t off = a.e.src_off + begin;
      if (off + (end - begin) <= a.e.src->size())
        p.data = std::make_shared<std::vector<uint8_t>>(a.e.src->begin() + off, a.e.src->begin() + off + (end - begin));
    }
    out_q_[vc].push_back(std::move(p));
    ++a.next_pkt;
  }
  pump_out(vc);
  if (a.next_pkt == a.seq_len) {
    // stream fully queued: local completion (send side) and next stream
    SendEntry done = a.e;
    a.active = false;
    if (done.cq >= 0) complete(done.cq, Completion{done.context, done.payload_len, node_, 0});
    pump_send(vc);
  } else {
    pump_send(vc);
  }
}

void Nic::pump_out(int vc) {
  if (out_busy_[vc] || out_q_[vc].empty()) return;
  out_busy_[vc] = true;
  const Time t = std::max(sim_.now(), net_.inject_free_at(node_));
  sim_.at(t, [this, vc]() {
    Packet p = std::move(out_q_[vc].front());
    out_q_[vc].pop_front();
    ++stats_.pkts_sent;
    stats_.bytes_sent += p.payload;
    net_.send(p);
    out_busy_[vc] = false;
    emit_packets(vc);   // queue space became available
    pump_out(vc);
  });
}

// ---- receive path ----------------------------------------------------------------------------
void Nic::on_packet(const Packet& p) {
  ++stats_.pkts_recv;
  stats_.bytes_recv += p.payload;
  if (p.kind == Packet::Barrier) {
    if (p.barrier_phase == 0) {
      if (bar_active_) { ++bar_children_in_; barrier_step(); } else ++bar_pending_fanin_;
    } else {
      if (bar_active_) { bar_got_fanout_ = true; barrier_step(); } else bar_pending_fanout_ = true;
    }
    return;
  }
  const uint64_t key = (static_cast<uint64_t>(p.src) << 32) | p.stream_id;
  if (p.first) on_stream_first(p);
  auto it = recv_.find(key);
  if (it == recv_.end()) return;   // stream was rejected
  stream_payload(it->second, p, key);
}

void Nic::on_stream_first(const Packet& p) {
  const uint64_t key = (static_cast<uint64_t>(p.src) << 32) | p.stream_id;
  RecvStream rs;
  rs.hdr = p.hdr;
  rs.src = p.src;
  rs.seq_len = p.seq_len;
  switch (p.hdr.type) {
    case StreamType::Msg: {
      RecvQueue* rq = nullptr;
      for (auto& q : rqs_) if (q.alive && q.key == p.hdr.key) rq = &q;
      if (rq == nullptr || rq->posted.empty() || rq->posted.front().len < p.hdr.length) {
        last_error = "node " + std::to_string(node_) + ": no matching receive for key " + std::to_string(p.hdr.key);
        return;
      }
      PostedRecv pr = rq->posted.front();
      rq->posted.pop_front();
      rs.dst = pr.buf;
      rs.dst_off = pr.off;
      rs.cq = rq->cq;
      rs.context = pr.context;
      break;
    }
    case StreamType::Write: {
      auto it = regions_.find(p.hdr.key);
      if (it == regions_.end()) {
        last_error = "node " + std::to_string(node_) + ": write to unregistered region " + std::to_string(p.hdr.key);
        return;
      }
      if (p.hdr.offset + p.hdr.length > it->second.len) {
        last_error = "node " + std::to_string(node_) + ": write beyond region " + std::to_string(p.hdr.key);
        return;
      }
      rs.dst = it->second.buf;
      rs.dst_off = it->second.off + p.hdr.offset;
      rs.complete_notify = false;
      break;
    }
    case StreamType::ReadReq: {
      auto it = regions_.find(p.hdr.key);
      if (it == regions_.end()) {
        last_error = "node " + std::to_string(node_) + ": read of unregistered region " + std::to_string(p.hdr.key);
        return;
      }
      SendEntry e;
      e.hdr.type = StreamType::ReadResp;
      e.hdr.length = p.hdr.read_len;
      e.hdr.key = p.hdr.resp_key;
      e.dst = p.src; e.vc = 1; e.cq = -1; e.context = 0;
      if (p.hdr.offset + p.hdr.read_len > it->second.len) {
        last_error = "node " + std::to_string(node_) + ": read beyond region " + std::to_string(p.hdr.key);
        return;
      }
      e.src = it->second.buf;
      e.src_off = it->second.off + p.hdr.offset;
      e.payload_len = p.hdr.read_len;
      start_send(std::move(e));
      rs.complete_notify = false;
      break;
    }
    case StreamType::ReadResp: {
      auto it = reads_.find(p.hdr.key);
      if (it == reads_.end()) {
        last_error = "node " + std::to_string(node_) + ": unexpected read response";
        return;
      }
      rs.dst = it->second.into;
      rs.dst_off = it->second.off;
      rs.cq = it->second.cq;
      rs.context = it->second.context;
      reads_.erase(it);
      break;
    }
  }
  ++stats_.streams_recv;
  recv_[key] = std::move(rs);
}

void Nic::stream_payload(RecvStream& rs, const Packet& p, uint64_t key) {
  const uint32_t data = p.payload - (p.first ? kStreamHdrBytes : 0);
  const uint64_t begin = p.seq == 0 ? 0 : (uint64_t)p.seq * kMtu - kStreamHdrBytes;
  if (p.data && rs.dst && rs.dst_off + begin + data <= rs.dst->size())
    std::memcpy(rs.dst->data() + rs.dst_off + begin, p.data->data(), data);
  rs.received += data;
  ++rs.got_pkts;
  // DMA-write the payload in 64-byte requests
  uint32_t left = data;
  const uint64_t total = rs.hdr.length;
  auto finish = [this, key]() {
    auto it = recv_.find(key);
    if (it == recv_.end()) return;
    RecvStream& r = it->second;
    if (r.written >= r.hdr.length && r.got_pkts == r.seq_len) {
      RecvStream done = r;
      recv_.erase(it);
      if (done.complete_notify) complete(done.cq, Completion{done.context, done.hdr.length, done.src, 0});
    }
  };
  if (total == 0 || data == 0) {
    sim_.after(p_.clock, finish);
    return;
  }
  while (left > 0) {
    const uint32_t n = std::min(left, p_.mem_req_bytes);
    left -= n;
    memq_.request(2, n, true, [this, key, n, finish]() {
      auto it = recv_.find(key);
      if (it != recv_.end()) it->second.written += n;
      finish();
    });
  }
}

// ---- barrier ---------------------------------------------------------------------------------
void Nic::send_barrier(int dst, int phase) {
  Packet p;
  p.kind = Packet::Barrier;
  p.src = node_; p.dst = dst; p.vc = 0;
  p.payload = 8;
  p.barrier_phase = phase;
  ++stats_.barrier_msgs_sent;
  ++stats_.pkts_sent;
  net_.send(p);
}

void Nic::barrier(std::function<void()> done) {
  submit([this, done]() {
    bar_active_ = true;
    bar_done_ = done;
    bar_children_in_ = bar_pending_fanin_;
    bar_pending_fanin_ = 0;
    bar_got_fanout_ = bar_pending_fanout_;
    bar_pending_fanout_ = false;
    barrier_step();
  });
}

void Nic::barrier_step() {
  if (!bar_active_) return;
  if (bar_children_in_ < (int)tree_.children.size()) return;   // wait for the fan-in of all children
  if (tree_.parent >= 0 && bar_children_in_ == (int)tree_.children.size() && !bar_got_fanout_) {
    if (bar_children_in_ >= 0) {
      // fan-in to the parent exactly once: mark by moving the counter past the child count
      send_barrier(tree_.parent, 0);
      bar_children_in_ = (int)tree_.children.size() + 1;
    }
    return;
  }
  if (tree_.parent >= 0 && !bar_got_fanout_) return;
  // root with all children in, or non-root that received the fan-out: release the subtree
  for (int c : tree_.children) send_barrier(c, 1);
  bar_active_ = false;
  bar_got_fanout_ = false;
  auto done = std::move(bar_done_);
  bar_done_ = nullptr;
  if (done) sim_.after(p_.host_poll_latency, done);
}

}  // namespace netsim
