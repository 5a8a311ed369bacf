// netsim: eager / rendezvous message passing and collectives on the RDMA library (see mpi.h).
#include "mpi.h"

#include <algorithm>
#include <cstring>

namespace netsim {

using abi::Addr;

namespace {
constexpr uint64_t kCtxShort = 1ull << 56, kCtxSend = 2ull << 56, kCtxRead = 3ull << 56, kCtxMask = (1ull << 56) - 1;
constexpr uint32_t kShortKey = 0xf00d;
constexpr uint32_t kBounceBuffers = 32;
}  // namespace

MiniMpi::MiniMpi(RdmaHost& host, MpiParams p) : host_(host), p_(p) {}

Co<void> MiniMpi::init() {
  if (co_await host_.init() != 0) throw std::runtime_error("rdma init failed");
  cq_ = co_await host_.create_cq(p_.cq_entries);
  if (cq_ < 0) throw std::runtime_error("mpi: no completion queue");
  rq_ = co_await host_.create_rq(kShortKey, cq_);
  if (rq_ < 0) throw std::runtime_error("mpi: no receive queue");
  short_stride_ = ((uint32_t)sizeof(Header) + p_.eager_limit + 63) / 64 * 64;
  short_bufs_ = host_.mem().alloc((uint64_t)p_.posted_recvs * short_stride_);
  for (uint32_t i = 0; i < p_.posted_recvs; ++i)
    co_await host_.recv_post(short_bufs_ + (uint64_t)i * short_stride_, short_stride_, rq_, kCtxShort | i);
  for (uint32_t i = 0; i < kBounceBuffers; ++i) bounce_free_.push_back(host_.mem().alloc(short_stride_));
  const int n = size();
  // Four buffers per peer is the least that cannot stall: data may use a peer's buffers down to the
  // last one, an explicit credit message goes out for every second buffer that was re-posted, and a
  // credit message frees only one buffer itself, so credit messages cannot chase each other.
  per_peer_credits_ = p_.posted_recvs / (uint32_t)std::max(1, n - 1);
  if (per_peer_credits_ < 4)
    throw std::runtime_error("mpi: posted_recvs must be at least 4 x (ranks - 1)");
  credits_.assign(n, (int)per_peer_credits_);
  owed_.assign(n, 0);
  co_await host_.barrier();   // every rank has posted its short-message buffers
}

Co<void> MiniMpi::finalize() {
  co_await barrier();
  while (!sends_in_flight_.empty()) co_await progress_one();
  co_await host_.barrier();
  co_await host_.fini();
}

// ---------------------------------------------------------------------------------------------
// progress engine
// ---------------------------------------------------------------------------------------------
Co<void> MiniMpi::progress_one() {
  const abi::RdmaCompletion e = co_await host_.read_comp(cq_);
  const uint64_t kind = e.context & ~kCtxMask;
  const uint32_t id = (uint32_t)(e.context & kCtxMask);
  if (kind == kCtxShort) {
    co_await handle_short(id);
  } else if (kind == kCtxSend) {
    auto it = sends_in_flight_.find(id);
    if (it != sends_in_flight_.end()) {
      bounce_free_.push_back(it->second.first);
      if (it->second.second) it->second.second->done = true;
      sends_in_flight_.erase(it);
    }
  } else if (kind == kCtxRead) {
    auto it = reads_.find(id);
    if (it != reads_.end()) {
      PendingRead pr = it->second;
      reads_.erase(it);
      pr.r->done = true;
      co_await send_control(kFin, pr.src, pr.sender_req);
    }
  }
}

Co<void> MiniMpi::handle_short(uint32_t i) {
  const Addr addr = short_bufs_ + (uint64_t)i * short_stride_;
  const Header h = host_.mem().load<Header>(addr);
  co_await host_.compute(p_.match_overhead);
  if (h.src < 0 || h.src >= size()) throw std::runtime_error("mpi: corrupt header");
  credits_[h.src] += (int)h.credits;
  if (h.kind == kEager || h.kind == kRts) {
    Req match;
    for (auto it = posted_.begin(); it != posted_.end(); ++it)
      if (matches(**it, h)) {
        match = *it;
        posted_.erase(it);
        break;
      }
    const uint8_t* payload = h.kind == kEager && h.len ? host_.mem().ptr(addr + sizeof(Header), h.len) : nullptr;
    if (match) {
      co_await deliver(h, payload, match);
    } else {
      ++stats_.unexpected;
      Unexpected u{h, {}};
      if (payload) {
        u.payload.assign(payload, payload + h.len);
        co_await copy_cost(h.len);
      }
      unexpected_.push_back(std::move(u));
    }
  } else if (h.kind == kFin) {
    auto it = rndv_sends_.find(h.req);
    if (it == rndv_sends_.end()) throw std::runtime_error("mpi: FIN for an unknown send");
    auto [req, key] = it->second;
    rndv_sends_.erase(it);
    co_await host_.memory_unreg(key);
    req->done = true;
  }
  // the buffer goes back to the NIC; its credit returns to the sender with the next header
  co_await host_.recv_post(addr, short_stride_, rq_, kCtxShort | i);
  ++owed_[h.src];
  if (owed_[h.src] >= per_peer_credits_ / 2 && credits_[h.src] >= 1)
    co_await send_control(kCredit, h.src, 0);
}

Co<void> MiniMpi::deliver(const Header& h, const uint8_t* payload, Req r) {
  const uint32_t n = std::min(h.len, r->len);
  r->src = h.src;
  r->received = n;
  if (h.kind == kEager) {
    if (n && payload) {
      auto [buf, off] = host_.mem().translate(r->buf, n);
      if (buf) std::memcpy(buf->data() + off, payload, n);
      co_await copy_cost(n);
    }
    r->done = true;
  } else {   // request-to-send: fetch the data from the sender's registered buffer
    const uint32_t id = next_id_++;
    reads_[id] = PendingRead{r, h.src, h.req};
    const int rc = co_await host_.memory_read(h.rkey, h.src, 0, r->buf, n, cq_, kCtxRead | id);
    if (rc != 0) throw std::runtime_error("mpi: rendezvous read refused");
  }
}

Co<void> MiniMpi::post_short(Header h, Addr payload, uint32_t len, int dst, Req done_flag) {
  // data may use the peer's buffers down to the last one, which is kept for control messages
  const int need = (h.kind == kEager || h.kind == kRts) ? 2 : 1;
  while (credits_[dst] < need) {
    ++stats_.credit_stalls;
    co_await progress_one();
  }
  --credits_[dst];
  while (bounce_free_.empty()) co_await progress_one();
  const Addr b = bounce_free_.back();
  bounce_free_.pop_back();
  h.credits = owed_[dst];
  owed_[dst] = 0;
  host_.mem().store(b, h);
  if (len) {
    auto [buf, off] = host_.mem().translate(payload, len);
    if (buf) std::memcpy(host_.mem().ptr(b + sizeof(Header), len), buf->data() + off, len);
    co_await copy_cost(len);
  }
  const uint32_t id = next_id_++;
  sends_in_flight_[id] = {b, done_flag};
  const int rc = co_await host_.send_post(b, (uint32_t)sizeof(Header) + len, dst, kShortKey, cq_, kCtxSend | id);
  if (rc != 0) throw std::runtime_error("mpi: send refused");
}

Co<void> MiniMpi::send_control(Kind kind, int dst, uint32_t req) {
  Header h{};
  h.kind = kind;
  h.src = rank();
  h.req = req;
  if (kind == kCredit) ++stats_.credit_msgs;
  co_await post_short(h, 0, 0, dst, nullptr);
}

// ---------------------------------------------------------------------------------------------
// point to point
// ---------------------------------------------------------------------------------------------
Co<MiniMpi::Req> MiniMpi::isend(Addr buf, uint32_t len, int dst, int tag) {
  if (dst < 0 || dst >= size()) throw std::invalid_argument("mpi: bad destination rank");
  Req r = std::make_shared<Request>();
  if (dst == rank()) {   // self send: straight into the matching logic
    Header h{};
    h.kind = kEager;
    h.src = rank();
    h.tag = tag;
    h.len = len;
    auto [sb, soff] = len ? host_.mem().translate(buf, len) : std::pair<Buffer, uint64_t>{nullptr, 0};
    const uint8_t* payload = sb ? sb->data() + soff : nullptr;
    Req match;
    for (auto it = posted_.begin(); it != posted_.end(); ++it)
      if (matches(**it, h)) {
        match = *it;
        posted_.erase(it);
        break;
      }
    if (match) {
      co_await deliver(h, payload, match);
    } else {
      Unexpected u{h, {}};
      if (payload) u.payload.assign(payload, payload + len);
      unexpected_.push_back(std::move(u));
    }
    r->done = true;
    co_return r;
  }
  Header h{};
  h.src = rank();
  h.tag = tag;
  h.len = len;
  if (len <= p_.eager_limit) {
    h.kind = kEager;
    ++stats_.eager_sent;
    co_await post_short(h, buf, len, dst, nullptr);
    r->done = true;   // the payload sits in a bounce buffer: the user buffer is free again
  } else {
    const uint32_t key = next_key_++, id = next_id_++;
    if (co_await host_.memory_reg(key, buf, len) != 0) throw std::runtime_error("mpi: cannot register the send buffer");
    rndv_sends_[id] = {r, key};
    h.kind = kRts;
    h.rkey = key;
    h.req = id;
    ++stats_.rndv_sent;
    co_await post_short(h, 0, 0, dst, nullptr);
  }
  co_return r;
}

Co<MiniMpi::Req> MiniMpi::irecv(Addr buf, uint32_t len, int src, int tag) {
  Req r = std::make_shared<Request>();
  r->src = src;
  r->tag = tag;
  r->buf = buf;
  r->len = len;
  for (auto it = unexpected_.begin(); it != unexpected_.end(); ++it)
    if (matches(*r, it->h)) {
      Unexpected u = std::move(*it);
      unexpected_.erase(it);
      co_await deliver(u.h, u.payload.empty() ? nullptr : u.payload.data(), r);
      co_return r;
    }
  posted_.push_back(r);
  co_return r;
}

Co<void> MiniMpi::wait(Req r) {
  while (!r->done) co_await progress_one();
}

Co<void> MiniMpi::send(Addr buf, uint32_t len, int dst, int tag) {
  Req r = co_await isend(buf, len, dst, tag);
  co_await wait(r);
}

Co<void> MiniMpi::recv(Addr buf, uint32_t len, int src, int tag) {
  Req r = co_await irecv(buf, len, src, tag);
  co_await wait(r);
}

Co<void> MiniMpi::sendrecv(Addr sbuf, uint32_t slen, int dst, int stag, Addr rbuf, uint32_t rlen, int src, int rtag) {
  Req rr = co_await irecv(rbuf, rlen, src, rtag);
  Req sr = co_await isend(sbuf, slen, dst, stag);
  co_await wait(rr);
  co_await wait(sr);
}

// ---------------------------------------------------------------------------------------------
// collectives
// ---------------------------------------------------------------------------------------------
void MiniMpi::add_i32(Addr acc, Addr in, uint32_t count) {
  if (!count) return;
  auto* a = reinterpret_cast<int32_t*>(host_.mem().ptr(acc, (uint64_t)count * 4));
  const auto* b = reinterpret_cast<const int32_t*>(host_.mem().ptr(in, (uint64_t)count * 4));
  for (uint32_t i = 0; i < count; ++i) a[i] += b[i];
}

Co<void> MiniMpi::barrier() {   // dissemination
  if (p_.coll_overhead) co_await host_.compute(p_.coll_overhead);
  const int n = size(), me = rank(), tag = coll_tag_ + 1;
  for (int d = 1; d < n; d <<= 1) co_await sendrecv(0, 0, (me + d) % n, tag, 0, 0, (me - d + n) % n, tag);
}

Co<void> MiniMpi::bcast(Addr buf, uint32_t len, int root) {   // binomial tree
  if (p_.coll_overhead) co_await host_.compute(p_.coll_overhead);
  const int n = size(), vr = (rank() - root + n) % n, tag = coll_tag_ + 2;
  int mask = 1;
  while (mask < n) {
    if (vr & mask) {
      co_await recv(buf, len, (vr - mask + root) % n, tag);
      break;
    }
    mask <<= 1;
  }
  mask >>= 1;
  while (mask > 0) {
    if (vr + mask < n) co_await send(buf, len, (vr + mask + root) % n, tag);
    mask >>= 1;
  }
}

Co<void> MiniMpi::reduce(Addr sbuf, Addr rbuf, uint32_t count, int root) {   // binomial tree, sum
  if (p_.coll_overhead) co_await host_.compute(p_.coll_overhead);
  const int n = size(), vr = (rank() - root + n) % n, tag = coll_tag_ + 3;
  const uint32_t bytes = count * 4;
  HostMemory& m = host_.mem();
  const Addr acc = m.alloc(std::max<uint32_t>(bytes, 4)), tmp = m.alloc(std::max<uint32_t>(bytes, 4));
  if (bytes) std::memcpy(m.ptr(acc, bytes), m.ptr(sbuf, bytes), bytes);
  co_await copy_cost(bytes);
  for (int mask = 1; mask < n; mask <<= 1) {
    if ((vr & mask) == 0) {
      const int peer = vr | mask;
      if (peer < n) {
        co_await recv(tmp, bytes, (peer + root) % n, tag);
        add_i32(acc, tmp, count);
        co_await host_.compute(bytes_time(bytes, p_.reduce_gbs * 1e9));
      }
    } else {
      co_await send(acc, bytes, ((vr & ~mask) + root) % n, tag);
      break;
    }
  }
  if (vr == 0 && bytes) std::memcpy(m.ptr(rbuf, bytes), m.ptr(acc, bytes), bytes);
  m.release(acc);
  m.release(tmp);
}

Co<void> MiniMpi::allreduce(Addr sbuf, Addr rbuf, uint32_t count) {
  if (p_.coll_overhead) co_await host_.compute(p_.coll_overhead);
  const int n = size(), me = rank(), tag = coll_tag_ + 4;
  const uint32_t bytes = count * 4;
  HostMemory& m = host_.mem();
  if ((n & (n - 1)) != 0) {   // not a power of two: reduce to rank 0, then broadcast
    co_await reduce(sbuf, rbuf, count, 0);
    co_await bcast(rbuf, bytes, 0);
    co_return;
  }
  const Addr tmp = m.alloc(std::max<uint32_t>(bytes, 4));
  if (bytes) std::memcpy(m.ptr(rbuf, bytes), m.ptr(sbuf, bytes), bytes);
  co_await copy_cost(bytes);
  for (int mask = 1; mask < n; mask <<= 1) {   // recursive doubling
    const int peer = me ^ mask;
    co_await sendrecv(rbuf, bytes, peer, tag, tmp, bytes, peer, tag);
    add_i32(rbuf, tmp, count);
    co_await host_.compute(bytes_time(bytes, p_.reduce_gbs * 1e9));
  }
  m.release(tmp);
}

Co<void> MiniMpi::reduce_scatter(Addr sbuf, Addr rbuf, uint32_t count) {   // pairwise exchange
  if (p_.coll_overhead) co_await host_.compute(p_.coll_overhead);
  const int n = size(), me = rank(), tag = coll_tag_ + 5;
  const uint32_t bytes = count * 4;
  HostMemory& m = host_.mem();
  const Addr tmp = m.alloc(std::max<uint32_t>(bytes, 4));
  if (bytes) std::memcpy(m.ptr(rbuf, bytes), m.ptr(sbuf + (uint64_t)me * bytes, bytes), bytes);
  co_await copy_cost(bytes);
  for (int i = 1; i < n; ++i) {
    const int dst = (me + i) % n, src = (me - i + n) % n;
    co_await sendrecv(sbuf + (uint64_t)dst * bytes, bytes, dst, tag, tmp, bytes, src, tag);
    add_i32(rbuf, tmp, count);
    co_await host_.compute(bytes_time(bytes, p_.reduce_gbs * 1e9));
  }
  m.release(tmp);
}

Co<void> MiniMpi::allgather(Addr sbuf, uint32_t len, Addr rbuf) {   // ring
  if (p_.coll_overhead) co_await host_.compute(p_.coll_overhead);
  const int n = size(), me = rank(), tag = coll_tag_ + 6;
  HostMemory& m = host_.mem();
  if (len) {
    auto [sb, so] = m.translate(sbuf, len);
    auto [rb, ro] = m.translate(rbuf + (uint64_t)me * len, len);
    if (sb && rb) std::memcpy(rb->data() + ro, sb->data() + so, len);
  }
  co_await copy_cost(len);
  const int right = (me + 1) % n, left = (me - 1 + n) % n;
  for (int i = 0; i < n - 1; ++i) {
    const int sblk = (me - i + n) % n, rblk = (me - i - 1 + n) % n;
    co_await sendrecv(rbuf + (uint64_t)sblk * len, len, right, tag, rbuf + (uint64_t)rblk * len, len, left, tag);
  }
}

Co<void> MiniMpi::alltoall(Addr sbuf, uint32_t len, Addr rbuf) {   // pairwise exchange
  if (p_.coll_overhead) co_await host_.compute(p_.coll_overhead);
  const int n = size(), me = rank(), tag = coll_tag_ + 7;
  HostMemory& m = host_.mem();
  if (len) {
    auto [sb, so] = m.translate(sbuf + (uint64_t)me * len, len);
    auto [rb, ro] = m.translate(rbuf + (uint64_t)me * len, len);
    if (sb && rb) std::memcpy(rb->data() + ro, sb->data() + so, len);
  }
  co_await copy_cost(len);
  for (int i = 1; i < n; ++i) {
    const int dst = (me + i) % n, src = (me - i + n) % n;
    co_await sendrecv(sbuf + (uint64_t)dst * len, len, dst, tag, rbuf + (uint64_t)src * len, len, src, tag);
  }
}

}  // namespace netsim
