#include "wire.h"

namespace tnnb {

static const char* kCmdNames[] = {
    "_START", "FORWARD_JOB", "BACKWARD_JOB", "BACKWARD_COMPLETE", "UPDATE_PARAMETERS", "TRAIN_MODE", "EVAL_MODE",
    "MODE_CHANGED", "SHUTDOWN", "CONFIG_TRANSFER", "CONFIG_RECEIVED", "LOAD_PARAMS", "PARAMS_LOADED", "SEND_PARAMS",
    "PARAMS_TRANSFER", "SAVE_TO_FILE", "STATUS_REQUEST", "STATUS_RESPONSE", "PARAMETERS_UPDATED", "HEALTH_CHECK",
    "PRINT_LR", "LR_PRINTED", "ERROR_REPORT", "JOB_FAILURE", "BARRIER_SYNC", "CHECKPOINT_REQUEST",
    "CHECKPOINT_COMPLETE", "UPDATE_LOAD", "REPORT_LOAD", "LOAD_REPORT", "START_PROFILING", "PROFILING_STARTED",
    "PRINT_PROFILING", "PROFILING_PRINTED", "CLEAR_PROFILING", "PROFILING_CLEARED", "REPORT_PROFILING",
    "PROFILING_REPORTED", "PRINT_LOGS", "LOGS_PRINTED", "HANDSHAKE", "HANDSHAKE_ACK"};

const char* command_name(uint16_t c) { return c < CMD_COUNT ? kCmdNames[c] : "UNKNOWN"; }

void write_packet_header(ByteWriter& w, const PacketHeader& h) {
  w.put<uint8_t>(h.version);
  w.put<uint8_t>(h.type);
  w.put<uint8_t>(h.little_endian);
  w.put<uint64_t>(h.packet_length);
  w.put<uint64_t>(h.msg_length);
  w.put<uint64_t>(h.msg_serial_id);
  w.put<uint32_t>(h.packet_offset);
  w.put<uint32_t>(h.total_packets);
  w.put<uint8_t>(h.compression);
}

PacketHeader read_packet_header(const char* p, size_t n) {
  if (n < PacketHeader::kSize) throw std::runtime_error("packet shorter than its 36-byte header");
  ByteReader r(p, n);
  PacketHeader h;
  h.version = r.get<uint8_t>();
  h.type = r.get<uint8_t>();
  h.little_endian = r.get<uint8_t>();
  r.set_swap((h.little_endian != 0) != host_is_little_endian());
  h.packet_length = r.get<uint64_t>();
  h.msg_length = r.get<uint64_t>();
  h.msg_serial_id = r.get<uint64_t>();
  h.packet_offset = r.get<uint32_t>();
  h.total_packets = r.get<uint32_t>();
  h.compression = r.get<uint8_t>();
  return h;
}

static void put_strings(ByteWriter& w, const std::vector<std::string>& v) {
  w.put<uint64_t>(v.size());
  for (const auto& s : v) w.str(s);
}
static std::vector<std::string> get_strings(ByteReader& r) {
  const uint64_t n = r.get<uint64_t>();
  std::vector<std::string> v;
  for (uint64_t i = 0; i < n; ++i) v.push_back(r.str());
  return v;
}

std::string serialize_message(const Message& m) {
  ByteWriter w;
  w.put<uint16_t>(m.command);
  w.put<uint32_t>(m.kind);
  switch (m.kind) {
    case PAYLOAD_NONE: break;
    case PAYLOAD_JOB:
      w.put<uint64_t>(m.job.pid);
      w.put<uint64_t>(m.job.tensors.size());
      for (const auto& kv : m.job.tensors) {
        w.str(kv.first);
        write_tensor(w, kv.second);
      }
      break;
    case PAYLOAD_STRING: w.str(m.text); break;
    case PAYLOAD_BOOL: w.put<uint8_t>(m.flag ? 1 : 0); break;
    case PAYLOAD_PROFILER:
      w.put<int64_t>(m.profiler.start_time);
      w.put<uint32_t>(static_cast<uint32_t>(m.profiler.events.size()));
      for (const auto& e : m.profiler.events) {
        w.put<int64_t>(e.start);
        w.put<int64_t>(e.end);
        w.put<uint8_t>(e.type);
        w.str(e.name);
        w.str(e.source);
      }
      break;
    case PAYLOAD_STAGE_CONFIG:
      w.str(m.stage.graph_state);
      put_strings(w, m.stage.input_uids);
      put_strings(w, m.stage.output_uids);
      w.str(m.stage.optimizer_config);
      w.str(m.stage.scheduler_config);
      w.str(m.stage.next_stage);
      w.str(m.stage.prev_stage);
      w.str(m.stage.coordinator);
      break;
    default: throw std::runtime_error("unknown payload kind");
  }
  return std::move(w.buf);
}

Message parse_message(const char* p, size_t n, bool swap_endian) {
  ByteReader r(p, n, swap_endian);
  Message m;
  m.command = r.get<uint16_t>();
  m.kind = r.get<uint32_t>();
  switch (m.kind) {
    case PAYLOAD_NONE: break;
    case PAYLOAD_JOB: {
      m.job.pid = r.get<uint64_t>();
      const uint64_t cnt = r.get<uint64_t>();
      for (uint64_t i = 0; i < cnt; ++i) {
        std::string uid = r.str();
        m.job.tensors.emplace_back(std::move(uid), read_tensor(r));
      }
      break;
    }
    case PAYLOAD_STRING: m.text = r.str(); break;
    case PAYLOAD_BOOL: m.flag = r.get<uint8_t>() != 0; break;
    case PAYLOAD_PROFILER: {
      m.profiler.start_time = r.get<int64_t>();
      const uint32_t cnt = r.get<uint32_t>();
      for (uint32_t i = 0; i < cnt; ++i) {
        ProfEvent e;
        e.start = r.get<int64_t>();
        e.end = r.get<int64_t>();
        e.type = r.get<uint8_t>();
        e.name = r.str();
        e.source = r.str();
        m.profiler.events.push_back(std::move(e));
      }
      break;
    }
    case PAYLOAD_STAGE_CONFIG:
      m.stage.graph_state = r.str();
      m.stage.input_uids = get_strings(r);
      m.stage.output_uids = get_strings(r);
      m.stage.optimizer_config = r.str();
      m.stage.scheduler_config = r.str();
      m.stage.next_stage = r.str();
      m.stage.prev_stage = r.str();
      m.stage.coordinator = r.str();
      break;
    default: throw std::runtime_error("unknown payload index " + std::to_string(m.kind));
  }
  return m;
}

std::vector<std::string> slice_message(const std::string& msg, uint64_t msg_id, uint64_t max_packet_size) {
  if (max_packet_size == 0) throw std::runtime_error("max_packet_size must be positive");
  const uint64_t total = msg.empty() ? 1 : (msg.size() + max_packet_size - 1) / max_packet_size;
  std::vector<std::string> out;
  out.reserve(total);
  for (uint64_t i = 0; i < total; ++i) {
    const uint64_t off = i * max_packet_size;
    const uint64_t len = std::min<uint64_t>(max_packet_size, msg.size() - off);
    PacketHeader h;
    h.little_endian = host_is_little_endian() ? 1 : 0;
    h.packet_length = len;
    h.msg_length = msg.size();
    h.msg_serial_id = msg_id;
    h.packet_offset = static_cast<uint32_t>(i);
    h.total_packets = static_cast<uint32_t>(total);
    ByteWriter w;
    write_packet_header(w, h);
    w.raw(msg.data() + off, len);
    out.push_back(std::move(w.buf));
  }
  return out;
}

char* Aggregator::reserve(const PacketHeader& h, bool* duplicate) {
  // Every field of the header comes from the peer: nothing is allocated or indexed before it has been checked
  // against the limits of this aggregator and against the other fields.
  if (h.total_packets == 0 || h.packet_offset >= h.total_packets) throw std::runtime_error("packet index out of range");
  if (h.msg_length > max_message_bytes_) throw std::runtime_error("message longer than this receiver accepts");
  if (h.total_packets > max_packets_) throw std::runtime_error("message split into more packets than this receiver accepts");
  if (h.packet_length > h.msg_length) throw std::runtime_error("fragment longer than its message");
  // a message of n bytes needs at most n packets (one byte each); an empty one exactly one
  if (h.total_packets > std::max<uint64_t>(h.msg_length, 1)) throw std::runtime_error("more packets than message bytes");
  // Every packet but the last carries the same payload size, so the byte
  // offset of packet i is i * (size of a non-final packet).
  uint64_t stride;
  if (h.total_packets == 1) stride = 0;
  else if (h.packet_offset + 1 < h.total_packets) stride = h.packet_length;
  else stride = (h.msg_length - h.packet_length) / (h.total_packets - 1);  // packet_length <= msg_length: no wrap
  // stride <= msg_length and packet_offset < total_packets <= msg_length <= max_message_bytes_ (< 2^63 / 2^32 is
  // not guaranteed), so multiply in 128 bits and compare before narrowing
  const unsigned __int128 off128 = static_cast<unsigned __int128>(stride) * h.packet_offset;
  if (off128 > h.msg_length || h.packet_length > h.msg_length - static_cast<uint64_t>(off128))
    throw std::runtime_error("fragment exceeds message length");
  const uint64_t off = static_cast<uint64_t>(off128);
  Slot& s = slots_[h.msg_serial_id];
  if (s.seen.empty()) {
    s.buf.resize(h.msg_length);
    s.seen.assign(h.total_packets, 0);
  }
  if (s.seen.size() != h.total_packets || s.buf.size() != h.msg_length) throw std::runtime_error("inconsistent fragments for one message");
  if (duplicate) *duplicate = s.seen[h.packet_offset] != 0;
  return s.buf.empty() ? nullptr : &s.buf[0] + off;
}

bool Aggregator::commit(const PacketHeader& h, std::string* out, uint64_t* msg_id) {
  auto it = slots_.find(h.msg_serial_id);
  if (it == slots_.end() || h.packet_offset >= it->second.seen.size()) throw std::runtime_error("commit of a packet that was not reserved");
  Slot& s = it->second;
  if (!s.seen[h.packet_offset]) {
    s.seen[h.packet_offset] = 1;
    ++s.received;
  }
  if (s.received == h.total_packets) {
    if (out) *out = std::move(s.buf);
    if (msg_id) *msg_id = h.msg_serial_id;
    slots_.erase(it);
    return true;
  }
  return false;
}

bool Aggregator::feed(const char* packet, size_t n, std::string* out, uint64_t* msg_id) {
  const PacketHeader h = read_packet_header(packet, n);
  if (n != PacketHeader::kSize + h.packet_length) throw std::runtime_error("packet length does not match its header");
  bool dup = false;
  char* dst = reserve(h, &dup);
  if (!dup && h.packet_length) std::memcpy(dst, packet + PacketHeader::kSize, h.packet_length);
  return commit(h, out, msg_id);
}

}  // namespace tnnb
