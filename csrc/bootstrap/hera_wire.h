// Hera-Core wire format.  Byte-compatible with the reference control plane
// (reference: src/hera/hera_msg.h:7-50): a 12-byte packed header
// {u32 magic 'HERA', u8 type, u8 version = 1, u16 reserved = 0, u32 payload_len}
// in host byte order, REGISTER_REQ {char hostname[64]; int pid} (68 B) and
// REGISTER_RESP {int rank; int world_size; char root_ip[64]} (72 B).
// TOPOLOGY_INIT/ACK, HEARTBEAT and GLOBAL_ABORT are reserved but unimplemented
// in the reference; here HEARTBEAT and GLOBAL_ABORT are live, and
// TOPOLOGY_INIT/ACK carry the ring neighbours on request.
#pragma once
#include <cstdint>

namespace mnccl {
namespace hera {

constexpr uint32_t kMagic = 0x48455241u;  // 'H''E''R''A'
constexpr uint8_t kVersion = 1;
constexpr int kDefaultPort = 9999;
constexpr uint32_t kMaxPayload = 1u << 20;  // sanity bound (the reference trusts payload_len)

enum class MsgType : uint8_t {
  RegisterReq = 0x01,
  RegisterResp = 0x02,
  TopologyInit = 0x03,
  TopologyAck = 0x04,
  Heartbeat = 0x05,
  GlobalAbort = 0xFF
};

#pragma pack(push, 1)
struct Header {
  uint32_t magic;
  uint8_t msg_type;
  uint8_t version;
  uint16_t reserved;
  uint32_t payload_len;
};
struct RegisterReq {
  char hostname[64];
  int32_t pid;
};
struct RegisterResp {
  int32_t rank;
  int32_t world_size;
  char root_ip[64];
};
struct TopologyInfo {
  int32_t prev_rank;
  int32_t next_rank;
  char next_ip[64];
  int32_t next_port;
};
struct Heartbeat {
  int32_t rank;
  uint32_t state;      // 0 = healthy, 1 = error seen locally
  uint32_t timestamp;  // seconds, sender's monotonic clock
};
struct GlobalAbort {
  int32_t origin_rank;
  uint32_t reason;
};
#pragma pack(pop)

static_assert(sizeof(Header) == 12, "Hera header is 12 bytes on the wire");
static_assert(sizeof(RegisterReq) == 68, "REGISTER_REQ is 68 bytes on the wire");
static_assert(sizeof(RegisterResp) == 72, "REGISTER_RESP is 72 bytes on the wire");
static_assert(sizeof(TopologyInfo) == 76, "TopologyInfo is 76 bytes on the wire");
static_assert(sizeof(Heartbeat) == 12, "Heartbeat is 12 bytes on the wire");

}  // namespace hera
}  // namespace mnccl
