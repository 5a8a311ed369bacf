// netsim: RDMA NIC model and the host-side API of a simulated node.
//
// Mirrors the structure of the reference's NIC (rdmaNic.h / rdmaNic*.h): a command queue fed by
// the host, a send engine that DMA-reads the source buffer in 64-byte requests and packs the data
// into MTU-sized packets, a receive engine that matches incoming streams against posted receives,
// registered memory regions or outstanding reads and DMA-writes the payload, a memory request
// queue with three source channels, round-robin arbitration, a global limit of outstanding
// requests and fences, per-VC network output queues, completion queues written back to host
// memory, and a k-ary tree barrier.
#pragma once
#include <deque>
#include <map>
#include <unordered_map>

#include "sim.h"

namespace netsim {

struct NicParams {
  uint32_t cmd_q_size = 64;        // rdmaNic.cc:32-126 defaults
  uint32_t max_mem_reqs = 128;
  uint32_t mem_req_bytes = 64;
  uint32_t barrier_degree = 4;
  uint32_t num_vcs = 2;
  uint32_t out_q_depth = 32;
  uint32_t send_ready_depth = 16;  // packets a send stream may have ready (rdmaNicSendEngine.cc:24)
  Time clock = 1 * kNs;            // 1 GHz
  Time mem_latency = 80 * kNs;     // host memory round trip seen by the NIC
  double mem_bw = 100e9;           // bytes/s of the NIC's DMA path
  Time host_cmd_latency = 150 * kNs;  // MMIO write of one 64-byte command
  Time host_poll_latency = 50 * kNs;  // host noticing a completion entry
};

// ---------------------------------------------------------------------------------------------
// Memory request queue: channels 0 (completion-tail writes), 1 (responses), 2 (DMA)
// ---------------------------------------------------------------------------------------------
class MemRequestQ {
 public:
  MemRequestQ(Simulator& sim, const NicParams& p) : sim_(sim), p_(p), chan_(3) {}
  // Queues one request of `bytes` (<= mem_req_bytes) on `channel`; `done` runs when it completes.
  void request(int channel, uint32_t bytes, bool is_write, std::function<void()> done);
  // Later requests of `channel` start only after every earlier request of that channel finished.
  void fence(int channel);
  uint64_t issued() const { return issued_; }
  uint32_t max_pending_seen() const { return max_seen_; }
  std::vector<int> issue_order;  // channel of every issued request, in order (kept for tests)
  bool record_order = false;

 private:
  struct Req {
    uint32_t bytes;
    bool write, is_fence;
    std::function<void()> done;
  };
  struct Chan {
    std::deque<Req> q;
    uint32_t inflight = 0;
  };
  void pump();
  Simulator& sim_;
  const NicParams& p_;
  std::vector<Chan> chan_;
  uint32_t pending_ = 0, max_seen_ = 0;
  int rr_ = 0;
  Time port_free_ = 0;
  uint64_t issued_ = 0;
};

// ---------------------------------------------------------------------------------------------
// k-ary tree rooted at node 0 (rdmaNicTree.h)
// ---------------------------------------------------------------------------------------------
struct Tree {
  Tree(int node, int n, int degree);
  int parent = -1;
  std::vector<int> children;
};

struct Completion {
  uint64_t context = 0;
  uint32_t length = 0;
  int src_node = -1;
  Time time = 0;
};

struct NicStats {
  uint64_t pkts_sent = 0, pkts_recv = 0, bytes_sent = 0, bytes_recv = 0, streams_sent = 0, streams_recv = 0,
           barrier_msgs_sent = 0, commands = 0;
};

using Buffer = std::shared_ptr<std::vector<uint8_t>>;

class Nic {
 public:
  Nic(Simulator& sim, Network& net, int node, NicParams p);

  // ---- host API (the reference's librdma, tests/app/rdma/include/rdma.h:30-69) ----
  int node() const { return node_; }
  int num_nodes() const { return net_.nodes(); }
  // Buffers are whole allocations; the trailing `*_off` arguments select where inside the
  // allocation the transfer starts (a host program passes addresses, see host.h).
  int create_cq();
  int create_rq(uint32_t key, int cq);
  bool destroy_cq(int cq);      // false: unknown id or still referenced by a receive queue
  bool destroy_rq(int rq);
  void fini();                  // later commands are refused (last_error is set)
  void recv_post(Buffer buf, uint32_t len, int rq, uint64_t context, uint64_t buf_off = 0);
  void send_post(Buffer buf, uint32_t len, int dst, uint32_t rq_key, int cq, uint64_t context,
                 uint64_t buf_off = 0);
  void memory_reg(uint32_t key, Buffer buf, uint64_t buf_off = 0, uint64_t len = ~0ull);
  void memory_unreg(uint32_t key);
  void memory_write(uint32_t key, int dst, uint64_t offset, Buffer data, uint32_t len, int cq, uint64_t context,
                    uint64_t data_off = 0);
  void memory_read(uint32_t key, int dst, uint64_t offset, Buffer into, uint32_t len, int cq, uint64_t context,
                   uint64_t into_off = 0);
  // A front end that models the MMIO command ring itself (host.h) switches the built-in
  // command latency off and receives completion entries instead of the internal queues.
  void set_direct(bool on) { direct_ = on; }
  void set_cq_sink(std::function<void(int cq, const Completion&)> fn) { cq_sink_ = std::move(fn); }
  Simulator& sim() { return sim_; }
  const NicParams& params() const { return p_; }
  // Calls `fn` (once) as soon as the CQ has an entry; entries are delivered in completion order.
  void on_completion(int cq, std::function<void(const Completion&)> fn);
  void barrier(std::function<void()> done);

  const NicStats& stats() const { return stats_; }
  MemRequestQ& memq() { return memq_; }
  std::string last_error;

 private:
  struct SendEntry {
    StreamHdr hdr;
    int dst, vc, cq;           // cq < 0: no local completion
    uint64_t context;
    Buffer src;                // bytes to send (may be null: size-only traffic)
    uint64_t src_off = 0;
    uint32_t payload_len;      // bytes DMA-read from src (0 for ReadReq)
  };
  struct RecvStream {
    StreamHdr hdr;
    int src;
    uint32_t seq_len, got_pkts = 0;
    uint64_t written = 0, received = 0;
    Buffer dst;
    uint64_t dst_off = 0;
    int cq = -1;
    uint64_t context = 0;
    bool complete_notify = true;
  };
  struct PostedRecv {
    Buffer buf;
    uint32_t len;
    uint64_t context;
    uint64_t off = 0;
  };
  struct RecvQueue {
    uint32_t key;
    int cq;
    std::deque<PostedRecv> posted;
    bool alive = true;
  };
  struct Region {
    Buffer buf;
    uint64_t off = 0, len = ~0ull;
  };
  struct CompQueue {
    std::deque<Completion> entries;
    std::deque<std::function<void(const Completion&)>> waiters;
    bool alive = true;
  };

  void submit(std::function<void()> cmd);   // host -> command queue -> NIC
  void start_send(SendEntry e);
  void pump_send(int vc);
  void emit_packets(int vc);
  void pump_out(int vc);
  void on_packet(const Packet& p);
  void on_stream_first(const Packet& p);
  void stream_payload(RecvStream& rs, const Packet& p, uint64_t key);
  void complete(int cq, Completion c);
  void barrier_step();
  void send_barrier(int dst, int phase);

  Simulator& sim_;
  Network& net_;
  int node_;
  NicParams p_;
  MemRequestQ memq_;
  NicStats stats_;
  Tree tree_;
  uint64_t next_stream_ = 1;
  uint32_t next_resp_key_ = 1;
  Time cmd_free_ = 0;
  uint32_t cmds_in_flight_ = 0;

  struct ActiveSend {
    SendEntry e;
    uint64_t stream_id;
    uint32_t seq_len, next_pkt = 0;     // next packet to emit
    uint64_t read_issued = 0, read_done = 0;
    uint32_t ready_pkts = 0;            // packets whose data has been read but not queued
    bool active = false;
  };
  std::vector<std::deque<SendEntry>> send_fifo_;   // per VC
  std::vector<ActiveSend> active_;                 // per VC
  std::vector<std::deque<Packet>> out_q_;          // per VC
  std::vector<bool> out_busy_;
  std::unordered_map<uint64_t, RecvStream> recv_;  // key: (src << 32) | stream id
  std::vector<RecvQueue> rqs_;
  std::vector<CompQueue> cqs_;
  std::map<uint32_t, Region> regions_;
  struct PendingRead {
    Buffer into;
    int cq;
    uint64_t context;
    uint64_t off = 0;
  };
  bool direct_ = false, finished_ = false;
  std::function<void(int, const Completion&)> cq_sink_;
  std::map<uint32_t, PendingRead> reads_;
  // barrier state
  int bar_children_in_ = 0;
  bool bar_active_ = false, bar_got_fanout_ = false;
  int bar_pending_fanin_ = 0;      // fan-in messages that arrived before the local barrier call
  bool bar_pending_fanout_ = false;
  std::function<void()> bar_done_;
};

}  // namespace netsim
