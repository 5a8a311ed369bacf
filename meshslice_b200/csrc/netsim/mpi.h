// netsim: a small message-passing layer on the RDMA library, with the two protocols of the
// reference's MVAPICH2 channel for this NIC (tests/app/mpi/patch.diff: ch3_rdma.cpp, progress
// engine and rendezvous code):
//   eager       header + payload (up to `eager_limit` bytes) is copied into a bounce buffer and
//               sent with send_post into one of the receiver's pre-posted short-message buffers
//               (receive queue key 0xf00d);
//   rendezvous  the sender registers the user buffer as a memory region and sends a small
//               request-to-send; the receiver, once the receive is matched, reads the data with a
//               one-sided memory_read and answers with a FIN, after which the sender unregisters.
// Pre-posted buffers are protected by per-peer credits that ride on every header (an explicit
// credit message goes out when nothing else does).  Collectives are the textbook algorithms on
// top of point-to-point.  All calls are awaitable; one program per rank drives progress.
#pragma once
#include <deque>
#include <list>

#include "host.h"

namespace netsim {

struct MpiParams {
  uint32_t eager_limit = 4096;     // largest payload sent eagerly (RDMA_SHORT_LENGTH of the reference)
  uint32_t posted_recvs = 64;      // pre-posted short-message buffers per rank
  uint32_t cq_entries = 512;
  double copy_gbs = 20.0;          // memcpy speed of the simulated core (bounce-buffer copies)
  double reduce_gbs = 8.0;         // speed of the reduction loop
  Time match_overhead = 40 * kNs;  // matching one incoming header against the posted receives
  Time coll_overhead = 0;          // software cost of entering a collective (argument checks, algorithm choice)
};

struct MpiStats {
  uint64_t eager_sent = 0, rndv_sent = 0, credit_msgs = 0, unexpected = 0, credit_stalls = 0;
};

class MiniMpi {
 public:
  static constexpr int kAnySource = -1;
  struct Request {
    bool done = false;
    // receive side
    int src = 0, tag = 0;
    abi::Addr buf = 0;
    uint32_t len = 0, received = 0;
  };
  using Req = std::shared_ptr<Request>;

  explicit MiniMpi(RdmaHost& host, MpiParams p = {});
  int rank() const { return host_.node(); }
  int size() const { return host_.num_nodes(); }
  RdmaHost& host() { return host_; }
  const MpiStats& stats() const { return stats_; }
  double wtime() const { return host_.sim().now() * 1e-12; }

  Co<void> init();
  Co<void> finalize();

  Co<Req> isend(abi::Addr buf, uint32_t len, int dst, int tag);
  Co<Req> irecv(abi::Addr buf, uint32_t len, int src, int tag);
  Co<void> wait(Req r);
  Co<void> send(abi::Addr buf, uint32_t len, int dst, int tag);
  Co<void> recv(abi::Addr buf, uint32_t len, int src, int tag);
  Co<void> sendrecv(abi::Addr sbuf, uint32_t slen, int dst, int stag, abi::Addr rbuf, uint32_t rlen, int src, int rtag);

  Co<void> barrier();
  Co<void> bcast(abi::Addr buf, uint32_t len, int root);
  // reductions sum 32-bit integers; `count` elements
  Co<void> reduce(abi::Addr sbuf, abi::Addr rbuf, uint32_t count, int root);
  Co<void> allreduce(abi::Addr sbuf, abi::Addr rbuf, uint32_t count);
  Co<void> reduce_scatter(abi::Addr sbuf, abi::Addr rbuf, uint32_t count_per_rank);
  Co<void> allgather(abi::Addr sbuf, uint32_t len, abi::Addr rbuf);
  Co<void> alltoall(abi::Addr sbuf, uint32_t len, abi::Addr rbuf);

 private:
  enum Kind : uint32_t { kEager = 1, kRts = 2, kFin = 3, kCredit = 4 };
  struct Header {          // 32 bytes in front of every short message
    uint32_t kind;
    int32_t src, tag;
    uint32_t len;          // payload bytes (eager) or message bytes (RTS)
    uint32_t rkey;         // RTS: memory-region key of the sender's buffer
    uint32_t req;          // RTS / FIN: sender's request id
    uint32_t credits;      // short-message buffers the sender of this header has re-posted for the receiver
    uint32_t reserved;
  };
  static_assert(sizeof(Header) == 32);
  struct Unexpected {
    Header h;
    std::vector<uint8_t> payload;
  };
  Co<void> progress_one();                      // handle one completion entry (waits for it)
  Co<void> handle_short(uint32_t buf_index);
  Co<void> deliver(const Header& h, const uint8_t* payload, Req r);   // matched message -> request
  Co<void> send_control(Kind kind, int dst, uint32_t req);
  Co<void> post_short(Header h, abi::Addr payload, uint32_t len, int dst, Req done_flag);
  Future<Unit> copy_cost(uint64_t bytes) { return host_.compute(bytes_time(bytes, p_.copy_gbs * 1e9)); }
  void add_i32(abi::Addr acc, abi::Addr in, uint32_t count);
  bool matches(const Request& r, const Header& h) const {
    return (r.src == kAnySource || r.src == h.src) && r.tag == h.tag;
  }

  RdmaHost& host_;
  MpiParams p_;
  MpiStats stats_;
  int cq_ = -1, rq_ = -1;
  abi::Addr short_bufs_ = 0;                    // posted_recvs x (header + eager_limit)
  uint32_t short_stride_ = 0;
  std::vector<abi::Addr> bounce_free_;          // bounce buffers for outgoing short messages
  std::map<uint32_t, std::pair<abi::Addr, Req>> sends_in_flight_;   // send context -> (bounce, request)
  std::map<uint32_t, std::pair<Req, uint32_t>> rndv_sends_;   // request id -> (request, region key), waiting for FIN
  struct PendingRead { Req r; int src; uint32_t sender_req; };
  std::map<uint32_t, PendingRead> reads_;       // read id -> matched receive
  std::list<Req> posted_;                       // receives not yet matched
  std::list<Unexpected> unexpected_;
  std::vector<int> credits_;                    // short messages this rank may still send to each peer
  std::vector<uint32_t> owed_;                  // buffers re-posted since the last header to each peer
  uint32_t per_peer_credits_ = 0;
  uint32_t next_id_ = 1, next_key_ = 0x1000;
  int coll_tag_ = 1 << 20;                      // tags of collectives live above the user's
};

}  // namespace netsim
