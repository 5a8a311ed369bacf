// netsim: process memory, the awaitable RDMA library and the NIC's command-ring front end.
#include "host.h"

#include <cstring>

namespace netsim {

using abi::Addr;
using abi::NicCmd;
using abi::NicResp;
using abi::RdmaCmd;

// =============================================================================================
// HostMemory
// =============================================================================================
Addr HostMemory::alloc(uint64_t bytes, bool phantom) {
  const Addr base = next_;
  next_ += ((bytes + 4095) / 4096 + 1) * 4096;   // one unmapped page between allocations
  blocks_[base] = Block{bytes, phantom ? nullptr : std::make_shared<std::vector<uint8_t>>(bytes)};
  allocated_ += bytes;
  return base;
}

void HostMemory::release(Addr base) {
  auto it = blocks_.find(base);
  if (it == blocks_.end()) throw std::out_of_range("release of an address that is not an allocation");
  allocated_ -= it->second.size;
  blocks_.erase(it);
}

std::pair<Buffer, uint64_t> HostMemory::translate(Addr addr, uint64_t len) const {
  auto it = blocks_.upper_bound(addr);
  if (it == blocks_.begin()) throw std::out_of_range("address below every allocation");
  --it;
  const uint64_t off = addr - it->first;
  if (off > it->second.size || len > it->second.size - off)
    throw std::out_of_range("range is not inside one allocation");
  return {it->second.buf, off};
}

uint8_t* HostMemory::ptr(Addr addr, uint64_t len) {
  auto [buf, off] = translate(addr, len);
  if (!buf) throw std::out_of_range("host access to phantom memory");
  return buf->data() + off;
}

// =============================================================================================
// RdmaHost: library side
// =============================================================================================
RdmaHost::RdmaHost(Nic& nic, HostParams hp)
    : nic_(nic), sim_(nic.sim()), hp_(hp), ring_(std::max<uint32_t>(2, nic.params().cmd_q_size)) {
  nic_.set_direct(true);   // the ring below accounts for the MMIO write of every command
  nic_.set_cq_sink([this](int cq, const Completion& c) { nic_completion(cq, c); });
}

Future<Unit> RdmaHost::compute(Time t) {
  Future<Unit> f;
  sim_.after(t, [f]() { f.set({}); });
  return f;
}

Co<int> RdmaHost::init() {
  co_await compute(hp_.call_overhead);
  resp_base_ = mem_.alloc(abi::kCmdSlots * sizeof(NicResp));
  head_shadow_ = mem_.alloc(64);
  mem_.store<uint32_t>(head_shadow_, 0);
  free_slots_.clear();
  for (int i = abi::kCmdSlots - 1; i >= 0; --i) free_slots_.push_back(i);
  // HostQueueInfo goes to the NIC as one MMIO write; the NIC reads it, sets its queues up and
  // writes NicQueueInfo back to host memory, which the host is polling
  const NicParams& np = nic_.params();
  co_await compute(np.host_cmd_latency + np.mem_latency + np.host_poll_latency);
  ready_ = true;
  co_return 0;
}

Co<NicResp> RdmaHost::command(NicCmd cmd) {
  if (!ready_) throw std::logic_error("rdma library used before init");
  co_await compute(hp_.call_overhead);
  while (free_slots_.empty()) {   // all response records are in use by commands in flight
    ++stats_.slot_waits;
    Future<Unit> f;
    slot_waiters_.push_back(f);
    co_await f;
  }
  const int slot = free_slots_.back();
  free_slots_.pop_back();
  cmd.resp_slot = (uint32_t)slot;
  mem_.store(resp_base_ + slot * sizeof(NicResp), NicResp{0, 0, 0, 0});
  while ((tail_ + 1) % ring_.size() == mem_.load<uint32_t>(head_shadow_)) {   // ring full
    ++stats_.ring_full_waits;
    Future<Unit> f;
    ring_waiters_.push_back(f);
    co_await f;
  }
  const uint32_t idx = tail_;
  ring_[idx] = cmd;
  tail_ = (tail_ + 1) % ring_.size();
  ++stats_.commands;
  Future<NicResp> done;
  resp_wait_[slot] = done;
  sim_.after(nic_.params().host_cmd_latency, [this, idx]() { nic_fetch(idx); });
  const NicResp r = co_await done;
  resp_wait_[slot].reset();
  free_slots_.push_back(slot);
  if (!slot_waiters_.empty()) {
    auto ws = std::move(slot_waiters_);
    slot_waiters_.clear();
    sim_.after(0, [ws]() { for (auto& w : ws) w.set({}); });
  }
  co_return r;
}

static int result_of(const NicResp& r) { return r.status != abi::kOk ? r.status : r.value; }

Co<int> RdmaHost::fini() {
  NicCmd c{};
  c.type = RdmaCmd::Fini;
  const NicResp r = co_await command(c);
  ready_ = false;
  co_return result_of(r);
}

Co<int> RdmaHost::barrier() {
  NicCmd c{};
  c.type = RdmaCmd::Barrier;
  co_return result_of(co_await command(c));
}

Co<int> RdmaHost::create_cq(uint32_t entries) {
  NicCmd c{};
  c.type = RdmaCmd::CreateCQ;
  c.u.create_cq.entries = entries;
  c.u.create_cq.ring_addr = mem_.alloc((uint64_t)entries * sizeof(abi::RdmaCompletion));
  c.u.create_cq.tail_addr = mem_.alloc(64);
  c.u.create_cq.head_addr = mem_.alloc(64);
  mem_.store<uint32_t>(c.u.create_cq.tail_addr, 0);
  mem_.store<uint32_t>(c.u.create_cq.head_addr, 0);
  const NicResp r = co_await command(c);
  if (r.status != abi::kOk) {
    mem_.release(c.u.create_cq.ring_addr);
    mem_.release(c.u.create_cq.tail_addr);
    mem_.release(c.u.create_cq.head_addr);
  }
  co_return result_of(r);
}

Co<int> RdmaHost::destroy_cq(int cq) {
  NicCmd c{};
  c.type = RdmaCmd::DestroyCQ;
  c.u.destroy.id = cq;
  const NicResp r = co_await command(c);
  if (r.status == abi::kOk) {
    auto it = cqs_.find(cq);
    if (it != cqs_.end()) {
      mem_.release(it->second.ring);
      mem_.release(it->second.tail_addr);
      mem_.release(it->second.head_addr);
      cqs_.erase(it);
    }
  }
  co_return result_of(r);
}

Co<int> RdmaHost::create_rq(uint32_t key, int cq) {
  NicCmd c{};
  c.type = RdmaCmd::CreateRQ;
  c.u.create_rq.key = key;
  c.u.create_rq.cq = cq;
  co_return result_of(co_await command(c));
}

Co<int> RdmaHost::destroy_rq(int rq) {
  NicCmd c{};
  c.type = RdmaCmd::DestroyRQ;
  c.u.destroy.id = rq;
  co_return result_of(co_await command(c));
}

Co<int> RdmaHost::send_post(Addr addr, uint32_t len, int dst_node, uint32_t rq_key, int cq, uint64_t context) {
  NicCmd c{};
  c.type = RdmaCmd::Send;
  c.u.send = abi::SendArgs{addr, len, dst_node, rq_key, cq, context};
  co_return result_of(co_await command(c));
}

Co<int> RdmaHost::recv_post(Addr addr, uint32_t len, int rq, uint64_t context) {
  NicCmd c{};
  c.type = RdmaCmd::Recv;
  c.u.recv = abi::RecvArgs{addr, len, rq, context};
  co_return result_of(co_await command(c));
}

Co<int> RdmaHost::memory_reg(uint32_t key, Addr addr, uint64_t len) {
  NicCmd c{};
  c.type = RdmaCmd::MemRgnReg;
  c.u.mem_reg = abi::MemRegArgs{key, 0, addr, len};
  co_return result_of(co_await command(c));
}

Co<int> RdmaHost::memory_unreg(uint32_t key) {
  NicCmd c{};
  c.type = RdmaCmd::MemRgnUnreg;
  c.u.mem_unreg.key = key;
  co_return result_of(co_await command(c));
}

Co<int> RdmaHost::memory_write(uint32_t key, int dst_node, uint64_t offset, Addr src, uint32_t len, int cq,
                               uint64_t context) {
  NicCmd c{};
  c.type = RdmaCmd::MemWrite;
  c.u.mem_write = abi::MemWriteArgs{key, dst_node, offset, src, len, cq, context};
  co_return result_of(co_await command(c));
}

Co<int> RdmaHost::memory_read(uint32_t key, int dst_node, uint64_t offset, Addr dst, uint32_t len, int cq,
                              uint64_t context) {
  NicCmd c{};
  c.type = RdmaCmd::MemRead;
  c.u.mem_read = abi::MemReadArgs{key, dst_node, offset, dst, len, cq, context};
  co_return result_of(co_await command(c));
}

bool RdmaHost::comp_ready(int cq) {
  auto it = cqs_.find(cq);
  if (it == cqs_.end() || !it->second.alive) return false;
  return mem_.load<uint32_t>(it->second.head_addr) != mem_.load<uint32_t>(it->second.tail_addr);
}

Co<abi::RdmaCompletion> RdmaHost::read_comp(int cq) {
  auto it = cqs_.find(cq);
  if (it == cqs_.end() || !it->second.alive) throw std::logic_error("read_comp on an unknown completion queue");
  for (;;) {
    CqRing& q = cqs_.at(cq);
    const uint32_t head = mem_.load<uint32_t>(q.head_addr), tail = mem_.load<uint32_t>(q.tail_addr);
    if (head != tail) {
      const auto e = mem_.load<abi::RdmaCompletion>(q.ring + head * sizeof(abi::RdmaCompletion));
      mem_.store<uint32_t>(q.head_addr, (head + 1) % q.entries);
      ++stats_.completions_read;
      co_return e;
    }
    ++stats_.empty_polls;
    if (q.waiter) throw std::logic_error("two programs wait on one completion queue");
    Future<Unit> f;
    q.waiter = f;
    co_await f;
  }
}

// =============================================================================================
// NIC side: command-ring front end
// =============================================================================================
void RdmaHost::nic_respond(uint32_t slot, int32_t value, int32_t status) {
  // response records travel on the response channel of the memory request queue
  nic_.memq().request(1, sizeof(NicResp), true, [this, slot, value, status]() {
    const NicResp r{value, status, 0, 1};
    mem_.store(resp_base_ + slot * sizeof(NicResp), r);
    if (resp_wait_[slot]) {
      Future<NicResp> f = *resp_wait_[slot];
      sim_.after(nic_.params().host_poll_latency, [f, r]() { f.set(r); });
    }
  });
}

void RdmaHost::nic_fetch(uint32_t idx) {
  const Time t = std::max(sim_.now(), fe_free_);
  fe_free_ = t + nic_.params().clock;
  sim_.at(t, [this, idx]() {
    NicCmd c;
    std::memcpy(&c, &ring_[idx], sizeof(c));
    nic_head_ = (idx + 1) % ring_.size();
    // the head index is mirrored into host memory so that the library sees ring space
    const uint32_t head = nic_head_;
    nic_.memq().request(0, 4, true, [this, head]() {
      mem_.store<uint32_t>(head_shadow_, head);
      if (!ring_waiters_.empty()) {
        auto ws = std::move(ring_waiters_);
        ring_waiters_.clear();
        sim_.after(nic_.params().host_poll_latency, [ws]() { for (auto& w : ws) w.set({}); });
      }
    });
    const uint32_t slot = c.resp_slot % abi::kCmdSlots;
    const int n = nic_.num_nodes();
    auto cq_ok = [&](int cq) { return cq < 0 || (cqs_.count(cq) && cqs_[cq].alive); };
    try {
      switch (c.type) {
        case RdmaCmd::CreateCQ: {
          int alive = 0;
          for (auto& kv : cqs_) alive += kv.second.alive;
          if (alive >= abi::kNumCompQ || c.u.create_cq.entries < 2) return nic_respond(slot, 0, abi::kNoResources);
          mem_.translate(c.u.create_cq.ring_addr, c.u.create_cq.entries * sizeof(abi::RdmaCompletion));
          const int id = nic_.create_cq();
          CqRing q;
          q.ring = c.u.create_cq.ring_addr;
          q.tail_addr = c.u.create_cq.tail_addr;
          q.head_addr = c.u.create_cq.head_addr;
          q.entries = c.u.create_cq.entries;
          q.alive = true;
          cqs_[id] = q;
          return nic_respond(slot, id, abi::kOk);
        }
        case RdmaCmd::DestroyCQ: {
          const int id = c.u.destroy.id;
          if (!cqs_.count(id) || !cqs_[id].alive || !nic_.destroy_cq(id)) return nic_respond(slot, 0, abi::kBadId);
          cqs_[id].alive = false;
          return nic_respond(slot, 0, abi::kOk);
        }
        case RdmaCmd::CreateRQ: {
          if (c.u.create_rq.cq < 0 || !cq_ok(c.u.create_rq.cq)) return nic_respond(slot, 0, abi::kBadId);
          return nic_respond(slot, nic_.create_rq(c.u.create_rq.key, c.u.create_rq.cq), abi::kOk);
        }
        case RdmaCmd::DestroyRQ:
          return nic_respond(slot, 0, nic_.destroy_rq(c.u.destroy.id) ? abi::kOk : abi::kBadId);
        case RdmaCmd::Send: {
          const auto& a = c.u.send;
          if (a.dst_node < 0 || a.dst_node >= n || !cq_ok(a.cq)) return nic_respond(slot, 0, abi::kBadId);
          auto [buf, off] = mem_.translate(a.addr, a.len);
          nic_.send_post(buf, a.len, a.dst_node, a.rq_key, a.cq, a.context, off);
          return nic_respond(slot, 0, abi::kOk);
        }
        case RdmaCmd::Recv: {
          const auto& a = c.u.recv;
          auto [buf, off] = mem_.translate(a.addr, a.len);
          nic_.recv_post(buf, a.len, a.rq, a.context, off);
          return nic_respond(slot, 0, abi::kOk);
        }
        case RdmaCmd::MemRgnReg: {
          const auto& a = c.u.mem_reg;
          auto [buf, off] = mem_.translate(a.addr, a.len);
          nic_.memory_reg(a.key, buf, off, a.len);
          return nic_respond(slot, 0, abi::kOk);
        }
        case RdmaCmd::MemRgnUnreg:
          nic_.memory_unreg(c.u.mem_unreg.key);
          return nic_respond(slot, 0, abi::kOk);
        case RdmaCmd::MemWrite: {
          const auto& a = c.u.mem_write;
          if (a.dst_node < 0 || a.dst_node >= n || !cq_ok(a.cq)) return nic_respond(slot, 0, abi::kBadId);
          auto [buf, off] = mem_.translate(a.src_addr, a.len);
          nic_.memory_write(a.key, a.dst_node, a.offset, buf, a.len, a.cq, a.context, off);
          return nic_respond(slot, 0, abi::kOk);
        }
        case RdmaCmd::MemRead: {
          const auto& a = c.u.mem_read;
          if (a.dst_node < 0 || a.dst_node >= n || a.cq < 0 || !cq_ok(a.cq)) return nic_respond(slot, 0, abi::kBadId);
          auto [buf, off] = mem_.translate(a.dst_addr, a.len);
          nic_.memory_read(a.key, a.dst_node, a.offset, buf, a.len, a.cq, a.context, off);
          return nic_respond(slot, 0, abi::kOk);
        }
        case RdmaCmd::Barrier:
          nic_.barrier([this, slot]() { nic_respond(slot, 0, abi::kOk); });
          return;
        case RdmaCmd::Fini:
          nic_.fini();
          return nic_respond(slot, 0, abi::kOk);
      }
      nic_respond(slot, 0, abi::kBadId);   // unknown command code
    } catch (const std::out_of_range&) {
      nic_respond(slot, 0, abi::kBadAddress);
    }
  });
}

void RdmaHost::nic_completion(int cq, const Completion& c) {
  auto it = cqs_.find(cq);
  if (it == cqs_.end() || !it->second.alive) return;
  CqRing& q = it->second;
  const uint32_t tail = mem_.load<uint32_t>(q.tail_addr), head = mem_.load<uint32_t>(q.head_addr);
  const uint32_t next = (tail + 1) % q.entries;
  if (next == head) {
    nic_.last_error = "node " + std::to_string(nic_.node()) + ": completion queue " + std::to_string(cq) + " overflow";
    return;
  }
  mem_.store(q.ring + tail * sizeof(abi::RdmaCompletion), abi::RdmaCompletion{c.context, c.length, c.src_node});
  mem_.store<uint32_t>(q.tail_addr, next);
  if (q.waiter) {
    Future<Unit> f = *q.waiter;
    q.waiter.reset();
    sim_.after(nic_.params().host_poll_latency, [f]() { f.set({}); });
  }
}

}  // namespace netsim
