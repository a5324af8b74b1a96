// Archiver wire format of the reference's coordinator/worker protocol, kept so
// that captured messages and StageConfig blobs stay parseable and so that the
// host control plane here speaks the same encoding (reference:
// include/distributed/{packet,message,job,stage_config,command_type,chunking,
// binary_serializer}.hpp, include/profiling/{event,profiler}.hpp).
//
//   PacketHeader (36 B) = u8 version ; u8 type ; u8 endianness(1 = little) ;
//       u64 packet_len ; u64 msg_len ; u64 msg_id ; u32 offset ; u32 total ; u8 compression
//   Message  = u16 command ; u32 payload index ; payload
//   payload  = 0 nothing | 1 Job | 2 string | 3 bool(u8) | 4 Profiler | 5 StageConfig
//   Job      = u64 pid ; u64 n ; n x { string uid ; TENSOR }
//   Profiler = i64 start ; u32 n ; n x { i64 start ; i64 end ; u8 type ; string name ; string source }
//   StageConfig = string graph_state ; strings input_uids ; strings output_uids ;
//       string optimizer ; string scheduler ; string next ; string prev ; string coordinator
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "bytes.h"
#include "tnng.h"

namespace tnnb {

enum CommandType : uint16_t {
  CMD_START = 0, FORWARD_JOB, BACKWARD_JOB, BACKWARD_COMPLETE, UPDATE_PARAMETERS, TRAIN_MODE, EVAL_MODE,
  MODE_CHANGED, SHUTDOWN, CONFIG_TRANSFER, CONFIG_RECEIVED, LOAD_PARAMS, PARAMS_LOADED, SEND_PARAMS,
  PARAMS_TRANSFER, SAVE_TO_FILE, STATUS_REQUEST, STATUS_RESPONSE, PARAMETERS_UPDATED, HEALTH_CHECK, PRINT_LR,
  LR_PRINTED, ERROR_REPORT, JOB_FAILURE, BARRIER_SYNC, CHECKPOINT_REQUEST, CHECKPOINT_COMPLETE, UPDATE_LOAD,
  REPORT_LOAD, LOAD_REPORT, START_PROFILING, PROFILING_STARTED, PRINT_PROFILING, PROFILING_PRINTED,
  CLEAR_PROFILING, PROFILING_CLEARED, REPORT_PROFILING, PROFILING_REPORTED, PRINT_LOGS, LOGS_PRINTED, HANDSHAKE,
  HANDSHAKE_ACK, CMD_COUNT
};
const char* command_name(uint16_t c);

struct PacketHeader {
  uint8_t version = 1;
  uint8_t type = 0;  // 0 data fragment, 1 prepare, 2 ready-to-write
  uint8_t little_endian = 1;
  uint64_t packet_length = 0;
  uint64_t msg_length = 0;
  uint64_t msg_serial_id = 0;
  uint32_t packet_offset = 0;
  uint32_t total_packets = 1;
  uint8_t compression = 0;
  static constexpr size_t kSize = 36;
};
void write_packet_header(ByteWriter& w, const PacketHeader& h);
PacketHeader read_packet_header(const char* p, size_t n);

struct Job {
  uint64_t pid = 0;
  std::vector<std::pair<std::string, HostTensor>> tensors;
};

struct ProfEvent {
  int64_t start = 0, end = 0;  // clock ticks (ns)
  uint8_t type = 0;            // 0 compute, 1 communication, 2 other
  std::string name, source;
};
struct ProfilerData {
  int64_t start_time = 0;
  std::vector<ProfEvent> events;
};

struct StageConfig {
  std::string graph_state;
  std::vector<std::string> input_uids, output_uids;
  std::string optimizer_config, scheduler_config, next_stage, prev_stage, coordinator;
};

enum PayloadKind : uint32_t { PAYLOAD_NONE = 0, PAYLOAD_JOB, PAYLOAD_STRING, PAYLOAD_BOOL, PAYLOAD_PROFILER, PAYLOAD_STAGE_CONFIG };

struct Message {
  uint16_t command = 0;
  uint32_t kind = PAYLOAD_NONE;
  Job job;
  std::string text;
  bool flag = false;
  ProfilerData profiler;
  StageConfig stage;
};

std::string serialize_message(const Message& m);
Message parse_message(const char* p, size_t n, bool swap_endian = false);

// Cut a serialized message into packets of at most max_packet_size payload
// bytes, each prefixed by its 36-byte header (offset = packet index).
std::vector<std::string> slice_message(const std::string& msg, uint64_t msg_id, uint64_t max_packet_size);

// Reassemble packets that may arrive in any order. feed() returns true (and
// fills `out`) when the message the packet belongs to is complete.
class Aggregator {
 public:
  // Limits on what a peer may make this receiver allocate: the longest message and the largest packet count it
  // accepts (defaults: 16 GiB and 2^22 packets - a 16 GiB message in 4 KiB packets). Headers beyond them, or
  // inconsistent with themselves, are rejected with an exception before any memory is touched.
  explicit Aggregator(uint64_t max_message_bytes = 16ull << 30, uint32_t max_packets = 1u << 22)
      : max_message_bytes_(max_message_bytes), max_packets_(max_packets) {}
  void set_limits(uint64_t max_message_bytes, uint32_t max_packets) {
    max_message_bytes_ = max_message_bytes;
    max_packets_ = max_packets;
  }
  bool feed(const char* packet, size_t n, std::string* out, uint64_t* msg_id = nullptr);
  // The two halves of feed() for a receiver that reads a payload straight from a socket into the message:
  // reserve() returns where the payload of the packet described by `h` belongs (`duplicate` tells whether that
  // packet has arrived before, in which case the caller must not write there), commit() records its arrival.
  // The message buffer does not move between the two calls, so several packets of one message may be filled at
  // the same time as long as reserve() and commit() themselves are serialised by the caller.
  char* reserve(const PacketHeader& h, bool* duplicate);
  bool commit(const PacketHeader& h, std::string* out, uint64_t* msg_id = nullptr);
  size_t pending() const { return slots_.size(); }

 private:
  struct Slot {
    std::string buf;
    std::vector<char> seen;
    uint32_t received = 0;
    uint64_t packet_size = 0;
  };
  std::map<uint64_t, Slot> slots_;
  uint64_t max_message_bytes_;
  uint32_t max_packets_;
};

}  // namespace tnnb
