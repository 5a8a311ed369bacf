// netsim: the host side of a simulated node: process memory, the user-space RDMA library and the
// command-ring front end of the NIC.
//
// Counterpart of the reference's librdma (tests/app/rdma/src/base.c:45-153, src/rdma.c:53-426,
// include/rdma.h:30-69) and of the MMIO command path of its NIC (rdmaNic.cc:145-227): `init`
// performs the queue-info handshake; every call encodes a 64-byte abi::NicCmd, waits for ring
// space, copies the record into the command ring and waits for the NIC's response record; the
// NIC front end decodes the record, translates host addresses, runs the command on the NIC
// model (nic.h) and writes the response through the NIC's memory request queue.  Completions are
// 16-byte entries that the NIC writes into completion rings in host memory; `read_comp` polls
// head != tail like the original.  Calls are awaitable (task.h) instead of blocking.
#pragma once
#include <array>
#include <cstring>
#include <map>
#include <optional>
#include <stdexcept>

#include "hostif.h"
#include "nic.h"
#include "task.h"

namespace netsim {

// Flat address space of one simulated process.  Allocations are the unit of translation: a
// transfer must lie inside one allocation.  "Phantom" allocations have a size but no bytes
// (bandwidth experiments that would otherwise copy gigabytes).
class HostMemory {
 public:
  abi::Addr alloc(uint64_t bytes, bool phantom = false);
  void release(abi::Addr base);
  // {buffer, offset inside it}; buffer is null for phantom memory.  Throws std::out_of_range.
  std::pair<Buffer, uint64_t> translate(abi::Addr addr, uint64_t len) const;
  uint8_t* ptr(abi::Addr addr, uint64_t len);   // host-side access; throws for phantom memory
  template <class T>
  T load(abi::Addr a) {
    T v;
    std::memcpy(&v, ptr(a, sizeof(T)), sizeof(T));
    return v;
  }
  template <class T>
  void store(abi::Addr a, const T& v) {
    std::memcpy(ptr(a, sizeof(T)), &v, sizeof(T));
  }
  uint64_t bytes_allocated() const { return allocated_; }

 private:
  struct Block {
    uint64_t size;
    Buffer buf;
  };
  std::map<abi::Addr, Block> blocks_;
  abi::Addr next_ = 0x10000000ull;
  uint64_t allocated_ = 0;
};

struct HostParams {
  Time call_overhead = 100 * kNs;   // CPU time of one library call before it touches the NIC
};

struct HostStats {
  uint64_t commands = 0, ring_full_waits = 0, slot_waits = 0, completions_read = 0, empty_polls = 0;
};

class RdmaHost {
 public:
  RdmaHost(Nic& nic, HostParams hp = {});
  RdmaHost(const RdmaHost&) = delete;

  HostMemory& mem() { return mem_; }
  Simulator& sim() { return sim_; }
  int node() const { return nic_.node(); }
  int num_nodes() const { return nic_.num_nodes(); }
  const HostStats& stats() const { return stats_; }
  Nic& nic() { return nic_; }

  // ---- the library (rdma.h of the reference); every call returns 0 / an id, or a negative abi status
  Co<int> init();
  Co<int> fini();
  Co<int> barrier();
  Co<int> create_cq(uint32_t entries = abi::kCompQSize);
  Co<int> destroy_cq(int cq);
  Co<int> create_rq(uint32_t key, int cq);
  Co<int> destroy_rq(int rq);
  Co<int> send_post(abi::Addr addr, uint32_t len, int dst_node, uint32_t rq_key, int cq, uint64_t context);
  Co<int> recv_post(abi::Addr addr, uint32_t len, int rq, uint64_t context);
  Co<int> memory_reg(uint32_t key, abi::Addr addr, uint64_t len);
  Co<int> memory_unreg(uint32_t key);
  Co<int> memory_write(uint32_t key, int dst_node, uint64_t offset, abi::Addr src, uint32_t len, int cq,
                       uint64_t context);
  Co<int> memory_read(uint32_t key, int dst_node, uint64_t offset, abi::Addr dst, uint32_t len, int cq,
                      uint64_t context);
  // Waits until the completion ring has an entry and pops it.
  Co<abi::RdmaCompletion> read_comp(int cq);
  bool comp_ready(int cq);                       // head != tail, no waiting
  // CPU time that is not NIC traffic (a memcpy, a reduction, application work).
  Future<Unit> compute(Time t);

 private:
  struct CqRing {
    abi::Addr ring = 0, tail_addr = 0, head_addr = 0;
    uint32_t entries = 0;
    bool alive = false;
    std::optional<Future<Unit>> waiter;   // a program sleeping in read_comp
  };
  Co<abi::NicResp> command(abi::NicCmd cmd);
  void nic_fetch(uint32_t ring_index);                       // NIC side: one command record arrived
  void nic_respond(uint32_t slot, int32_t value, int32_t status);
  void nic_completion(int cq, const Completion& c);          // NIC side: completion entry lands
  Nic& nic_;
  Simulator& sim_;
  HostParams hp_;
  HostMemory mem_;
  HostStats stats_;
  bool ready_ = false;
  // command ring (lives in the NIC's MMIO window) and its indices
  std::vector<abi::NicCmd> ring_;
  uint32_t tail_ = 0;                 // host: next slot to write
  uint32_t nic_head_ = 0;             // NIC: next slot to fetch
  abi::Addr head_shadow_ = 0;         // host memory word the NIC mirrors its head into
  abi::Addr resp_base_ = 0;           // kCmdSlots response records
  std::vector<int> free_slots_;
  std::array<std::optional<Future<abi::NicResp>>, abi::kCmdSlots> resp_wait_;
  std::vector<Future<Unit>> ring_waiters_, slot_waiters_;   // programs waiting for ring space / a response record
  Time fe_free_ = 0;                  // NIC front end: one command per clock
  std::map<int, CqRing> cqs_;
};

}  // namespace netsim
