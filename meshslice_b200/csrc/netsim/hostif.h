// netsim: the binary interface between a host process and its NIC.
//
// The counterpart of the reference's rdmaNicHostInterface.h:16-126: a host program talks to the
// NIC by writing fixed 64-byte command records into a command ring inside the NIC's MMIO window;
// the NIC answers every command by writing a response record into host memory (the flag word is
// the last field and is written last) and reports finished transfers as 16-byte entries of
// completion rings that also live in host memory.  The layouts below are this simulator's own;
// the sizes that matter for timing (64-byte commands, 16-byte completions, 16 completion queues
// of 32 entries) follow the reference.
#pragma once
#include <cstdint>

namespace netsim::abi {

using Addr = uint64_t;   // address in the simulated process

constexpr int kNumCompQ = 16;    // completion queues a process may create
constexpr int kCompQSize = 32;   // entries per completion ring
constexpr int kCmdSlots = 16;    // response records the host library cycles through

enum class RdmaCmd : uint32_t {
  Send = 1, Recv, Fini, CreateCQ, DestroyCQ, CreateRQ, DestroyRQ, MemRgnReg, MemRgnUnreg, MemWrite, MemRead, Barrier
};

struct SendArgs { Addr addr; uint32_t len; int32_t dst_node; uint32_t rq_key; int32_t cq; uint64_t context; };
struct RecvArgs { Addr addr; uint32_t len; int32_t rq; uint64_t context; };
struct CreateCqArgs { Addr ring_addr; Addr tail_addr; Addr head_addr; uint32_t entries; };
struct CreateRqArgs { uint32_t key; int32_t cq; };
struct DestroyArgs { int32_t id; };
struct MemRegArgs { uint32_t key; uint32_t reserved; Addr addr; uint64_t len; };
struct MemUnregArgs { uint32_t key; };
struct MemWriteArgs { uint32_t key; int32_t dst_node; uint64_t offset; Addr src_addr; uint32_t len; int32_t cq; uint64_t context; };
struct MemReadArgs { uint32_t key; int32_t dst_node; uint64_t offset; Addr dst_addr; uint32_t len; int32_t cq; uint64_t context; };

struct alignas(64) NicCmd {
  RdmaCmd type;
  uint32_t resp_slot;    // which response record the NIC answers into
  union {
    SendArgs send;
    RecvArgs recv;
    CreateCqArgs create_cq;
    CreateRqArgs create_rq;
    DestroyArgs destroy;
    MemRegArgs mem_reg;
    MemUnregArgs mem_unreg;
    MemWriteArgs mem_write;
    MemReadArgs mem_read;
  } u;
};
static_assert(sizeof(NicCmd) == 64, "a command is one 64-byte MMIO record");

struct RdmaCompletion {
  uint64_t context;
  uint32_t length;
  int32_t src_node;
};
static_assert(sizeof(RdmaCompletion) == 16, "completion entries are 16 bytes");

// Error codes of NicResp::status (0 = success).
enum : int32_t { kOk = 0, kBadId = -1, kBadAddress = -2, kNoResources = -3, kFinished = -4 };

struct NicResp {
  int32_t value;     // id of the created queue, else 0
  int32_t status;
  uint32_t reserved;
  uint32_t done;     // written last: the host polls this word
};
static_assert(sizeof(NicResp) == 16, "response records are 16 bytes");

// Setup handshake (rdmaNic.cc:145-202): the host tells the NIC where its response records
// live, the NIC tells the host where the command ring is and how large.
struct HostQueueInfo {
  Addr resp_addr;        // kCmdSlots response records
  Addr head_shadow_addr; // the NIC mirrors its ring head index here
};
struct NicQueueInfo {
  uint32_t ring_entries;
  uint32_t node_id, num_nodes;
  uint32_t ready;
};

}  // namespace netsim::abi
