// netsim: a stand-alone discrete-event model of an RDMA NIC and the network between nodes.
//
// It replaces the reference's network_simulator/ directory (an SST "rdmaNic" element that only
// builds inside an SST-elements tree with Vanadis RISC-V cores and the merlin router model) by a
// self-contained C++20 tool for offline analysis: the parts of the NIC that the reference owns
// (command queue, send / receive engines, memory request queue, network queues, tree barrier;
// rdmaNic.h:44-420) are modelled here, and what SST provided around them (cores, memory
// hierarchy, routers) is reduced to parametric latency / bandwidth models.  It is never on the
// training path.
//
// This header: simulation core (event queue) and network (links, torus and crossbar routing).
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <queue>
#include <string>
#include <vector>

namespace netsim {

using Time = uint64_t;  // picoseconds
constexpr Time kNs = 1000;
constexpr Time kUs = 1000 * kNs;

inline Time bytes_time(uint64_t bytes, double bytes_per_second) {
  return static_cast<Time>(static_cast<double>(bytes) / bytes_per_second * 1e12 + 0.5);
}

class Simulator {
 public:
  void at(Time t, std::function<void()> fn) { q_.push(Event{t < now_ ? now_ : t, seq_++, std::move(fn)}); }
  void after(Time dt, std::function<void()> fn) { at(now_ + dt, std::move(fn)); }
  Time now() const { return now_; }
  uint64_t events() const { return processed_; }
  // Runs until no event is left or `limit` events were processed.  Returns false on the limit.
  bool run(uint64_t limit = 2000000000ull) {
    while (!q_.empty()) {
      if (processed_ >= limit) return false;
      Event e = q_.top();
      q_.pop();
      now_ = e.t;
      ++processed_;
      e.fn();
    }
    return true;
  }

 private:
  struct Event {
    Time t;
    uint64_t seq;
    std::function<void()> fn;
    bool operator<(const Event& o) const { return t != o.t ? t > o.t : seq > o.seq; }
  };
  std::priority_queue<Event> q_;
  Time now_ = 0;
  uint64_t seq_ = 0, processed_ = 0;
};

// ---------------------------------------------------------------------------------------------
// packets
// ---------------------------------------------------------------------------------------------
enum class StreamType : uint8_t { Msg, Write, ReadReq, ReadResp };

// Header carried by the first packet of a stream (rdmaNic.h:296-309 has the reference's fields).
struct StreamHdr {
  StreamType type = StreamType::Msg;
  uint32_t length = 0;     // payload bytes of the whole stream
  uint32_t key = 0;        // receive-queue key, memory-region key or read-response key
  uint64_t offset = 0;     // offset inside the memory region (Write / ReadReq)
  uint32_t read_len = 0;   // ReadReq: bytes requested
  uint32_t resp_key = 0;   // ReadReq: key the response must carry
};
constexpr uint32_t kStreamHdrBytes = 32;   // bytes the header occupies in the first packet
constexpr uint32_t kMtu = 1024;            // NIC packet payload limit (rdmaNic.cc:29)
constexpr uint32_t kPktOverhead = 20;      // network header per packet (rdmaNicNetworkEvent.h:18-24)

struct Packet {
  enum Kind : uint8_t { Stream, Barrier } kind = Stream;
  int src = 0, dst = 0, vc = 0;
  uint32_t payload = 0;        // bytes after the network header (includes StreamHdr on packet 0)
  uint64_t stream_id = 0;
  uint32_t seq = 0, seq_len = 0;
  bool first = false;
  StreamHdr hdr;               // valid when first
  std::shared_ptr<std::vector<uint8_t>> data;  // optional real bytes of this packet
  int barrier_phase = 0;       // Barrier packets: 0 fan-in, 1 fan-out
};

inline uint32_t packets_for(uint32_t length) {   // ceil((hdr + len) / MTU), at least one
  uint32_t total = kStreamHdrBytes + length;
  return (total + kMtu - 1) / kMtu;
}

// ---------------------------------------------------------------------------------------------
// network
// ---------------------------------------------------------------------------------------------
struct LinkStats {
  uint64_t packets = 0, bytes = 0;
  Time busy = 0;
};

struct NetParams {
  double link_bw = 32e9;          // router-to-router, bytes/s (runVanadis.py:14-31: 32 GB/s)
  double nic_bw = 16e9;           // NIC-to-router (rdmaNic.py:110-113: 16 GB/s)
  Time link_latency = 10 * kNs;   // per hop
  Time router_latency = 20 * kNs; // input + output latency of a router
  uint32_t flit_bytes = 8;
};

class Network {
 public:
  using Deliver = std::function<void(const Packet&)>;
  Network(Simulator& sim, int nodes, NetParams p) : sim_(sim), n_(nodes), p_(p), sinks_(nodes) {}
  virtual ~Network() = default;
  int nodes() const { return n_; }
  void attach(int node, Deliver d) { sinks_[node] = std::move(d); }
  // Earliest time the NIC injection link of `node` is free (for output-queue back-pressure).
  Time inject_free_at(int node) const { return links_[inject_link(node)].free_at; }
  void send(const Packet& pkt);
  virtual std::string name() const = 0;
  const std::vector<LinkStats>& link_stats() const { return stats_; }
  uint64_t total_packets() const { return total_packets_; }
  int hops(int src, int dst) { return (int)route(src, dst).size(); }

 protected:
  struct Link {
    double bw;
    Time latency;
    Time free_at = 0;
  };
  int add_link(double bw, Time lat) {
    links_.push_back(Link{bw, lat});
    stats_.push_back(LinkStats{});
    return (int)links_.size() - 1;
  }
  virtual std::vector<int> route(int src, int dst) = 0;  // link ids, injection link first
  virtual int inject_link(int node) const = 0;
  Simulator& sim_;
  int n_;
  NetParams p_;
  std::vector<Link> links_;
  std::vector<LinkStats> stats_;

 private:
  void hop(std::shared_ptr<Packet> pkt, std::shared_ptr<std::vector<int>> path, size_t i);
  std::vector<Deliver> sinks_;
  uint64_t total_packets_ = 0;
};

// n-dimensional torus with dimension-order routing (the topology of runVanadis.py:42-64).
class Torus : public Network {
 public:
  Torus(Simulator& sim, std::vector<int> shape, NetParams p);
  std::string name() const override;
  std::vector<int> coords(int node) const;

 protected:
  std::vector<int> route(int src, int dst) override;
  int inject_link(int node) const override { return nic_up_[node]; }

 private:
  std::vector<int> shape_;
  std::vector<int> nic_up_, nic_down_;
  std::vector<std::vector<int>> plus_, minus_;  // [dim][node] -> link id
};

// Single non-blocking switch (NVSwitch-like): every node is two hops from every other node.
class Crossbar : public Network {
 public:
  Crossbar(Simulator& sim, int nodes, NetParams p);
  std::string name() const override { return "crossbar(" + std::to_string(n_) + ")"; }

 protected:
  std::vector<int> route(int src, int dst) override { return {up_[src], down_[dst]}; }
  int inject_link(int node) const override { return up_[node]; }

 private:
  std::vector<int> up_, down_;
};

std::unique_ptr<Network> make_network(Simulator& sim, const std::string& spec, int nodes, NetParams p);

}  // namespace netsim
