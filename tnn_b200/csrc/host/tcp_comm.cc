#include "tcp_comm.h"

#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <stdexcept>

namespace tnnb {
namespace {

bool read_exact(int fd, char* p, size_t n) {
  while (n) {
    ssize_t r = ::recv(fd, p, n, 0);
    if (r == 0) return false;
    if (r < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

bool write_exact(int fd, const char* p, size_t n) {
  while (n) {
    ssize_t r = ::send(fd, p, n, MSG_NOSIGNAL);
    if (r < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

void tune(int fd) {
  int one = 1;
  ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  // SO_SNDBUF / SO_RCVBUF stay untouched: an explicit size switches off the kernel's buffer auto-tuning and is
  // capped at net.core.{w,r}mem_max, which is far below what auto-tuning reaches on a fast link
}

std::string resolve_ipv4(const std::string& host) {
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  if (::getaddrinfo(host.c_str(), nullptr, &hints, &res) != 0 || !res) throw std::runtime_error("cannot resolve host " + host);
  char ip[INET_ADDRSTRLEN] = {0};
  ::inet_ntop(AF_INET, &reinterpret_cast<sockaddr_in*>(res->ai_addr)->sin_addr, ip, sizeof(ip));
  ::freeaddrinfo(res);
  return ip;
}

}  // namespace

TcpCommunicator::TcpCommunicator(std::string bind_host, int port, int sockets_per_endpoint, uint64_t max_packet_size)
    : host_(resolve_ipv4(bind_host)), port_(port), sockets_(sockets_per_endpoint < 1 ? 1 : sockets_per_endpoint),
      max_packet_(max_packet_size) {
  if (max_packet_ == 0) throw std::runtime_error("max_packet_size must be positive");
}

TcpCommunicator::~TcpCommunicator() { stop(); }

std::string TcpCommunicator::endpoint() const { return host_ + ":" + std::to_string(port_); }

int TcpCommunicator::start() {
  if (listen_fd_ >= 0) return port_;
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) throw std::runtime_error("socket() failed");
  int one = 1;
  ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons(static_cast<uint16_t>(port_));
  ::inet_pton(AF_INET, host_.c_str(), &a.sin_addr);
  if (::bind(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0 || ::listen(fd, 128) != 0) {
    const std::string why = std::strerror(errno);
    ::close(fd);
    throw std::runtime_error("cannot listen on " + endpoint() + ": " + why);
  }
  socklen_t len = sizeof(a);
  ::getsockname(fd, reinterpret_cast<sockaddr*>(&a), &len);
  port_ = ntohs(a.sin_port);
  listen_fd_ = fd;
  stopping_ = false;
  acceptor_ = std::thread([this] { accept_loop(); });
  return port_;
}

std::shared_ptr<TcpCommunicator::Peer> TcpCommunicator::peer_for(const std::string& name, bool create) {
  std::lock_guard<std::mutex> g(peers_mu_);
  auto it = peers_.find(name);
  if (it != peers_.end()) return it->second;
  if (!create) return nullptr;
  auto p = std::make_shared<Peer>();
  p->name = name;
  peers_[name] = p;
  return p;
}

void TcpCommunicator::adopt(int fd, const std::string& peer_name) {
  tune(fd);
  auto peer = peer_for(peer_name, true);
  auto c = std::make_shared<Conn>();
  c->fd = fd;
  c->peer = peer;
  {
    std::lock_guard<std::mutex> g(peer->mu);
    peer->conns.push_back(c);
  }
  {
    std::lock_guard<std::mutex> g(peers_mu_);
    all_conns_.push_back(c);
  }
  c->reader = std::thread([this, c] { read_loop(c); });
  c->writer = std::thread([this, c] { write_loop(c); });
}

void TcpCommunicator::accept_loop() {
  while (!stopping_) {
    pollfd p{listen_fd_, POLLIN, 0};
    int r = ::poll(&p, 1, 100);
    if (r <= 0) continue;
    sockaddr_in a{};
    socklen_t len = sizeof(a);
    int fd = ::accept(listen_fd_, reinterpret_cast<sockaddr*>(&a), &len);
    if (fd < 0) continue;
    // identity handshake: the peer's listening port, little-endian i32 (a peer that stays silent is dropped)
    timeval tv{5, 0};
    ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    unsigned char b[4];
    if (!read_exact(fd, reinterpret_cast<char*>(b), 4)) {
      ::close(fd);
      continue;
    }
    tv = timeval{0, 0};
    ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    const int32_t peer_port = static_cast<int32_t>(b[0] | (b[1] << 8) | (b[2] << 16) | (static_cast<uint32_t>(b[3]) << 24));
    char ip[INET_ADDRSTRLEN] = {0};
    ::inet_ntop(AF_INET, &a.sin_addr, ip, sizeof(ip));
    adopt(fd, std::string(ip) + ":" + std::to_string(peer_port));
  }
}

std::string TcpCommunicator::connect(const std::string& host, int port, double timeout_s) {
  const std::string ip = resolve_ipv4(host);
  const std::string name = ip + ":" + std::to_string(port);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s);
  for (int i = 0; i < sockets_; ++i) {
    int fd = -1;
    for (;;) {  // the peer's server may still be starting: retry until the deadline
      fd = ::socket(AF_INET, SOCK_STREAM, 0);
      if (fd < 0) throw std::runtime_error("socket() failed");
      sockaddr_in a{};
      a.sin_family = AF_INET;
      a.sin_port = htons(static_cast<uint16_t>(port));
      ::inet_pton(AF_INET, ip.c_str(), &a.sin_addr);
      if (::connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) == 0) break;
      ::close(fd);
      fd = -1;
      if (stopping_ || std::chrono::steady_clock::now() > deadline) throw std::runtime_error("cannot connect to " + name);
      std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
    const uint32_t p = static_cast<uint32_t>(port_);
    const unsigned char b[4] = {static_cast<unsigned char>(p), static_cast<unsigned char>(p >> 8),
                                static_cast<unsigned char>(p >> 16), static_cast<unsigned char>(p >> 24)};
    if (!write_exact(fd, reinterpret_cast<const char*>(b), 4)) {
      ::close(fd);
      throw std::runtime_error("handshake with " + name + " failed");
    }
    adopt(fd, name);
  }
  return name;
}

bool TcpCommunicator::connected(const std::string& endpoint) {
  auto p = peer_for(endpoint, false);
  if (!p) return false;
  std::lock_guard<std::mutex> g(p->mu);
  for (auto& c : p->conns)
    if (!c->closed) return true;
  return false;
}

std::vector<std::string> TcpCommunicator::peers() {
  std::lock_guard<std::mutex> g(peers_mu_);
  std::vector<std::string> out;
  for (auto& kv : peers_) out.push_back(kv.first);
  return out;
}

void TcpCommunicator::send(const std::string& endpoint, std::string message) {
  auto body = std::make_shared<const std::string>(std::move(message));
  send_view(endpoint, body->data(), body->size(), body);
}

void TcpCommunicator::send_view(const std::string& endpoint, const char* data, size_t n, std::shared_ptr<const void> keep) {
  auto peer = peer_for(endpoint, false);
  if (!peer) throw std::runtime_error("no connection to " + endpoint);
  const uint64_t id = next_msg_id_++;
  const uint64_t total = n == 0 ? 1 : (n + max_packet_ - 1) / max_packet_;
  std::lock_guard<std::mutex> g(peer->mu);
  std::vector<std::shared_ptr<Conn>> live;
  for (auto& c : peer->conns)
    if (!c->closed) live.push_back(c);
  if (live.empty()) throw std::runtime_error("connection to " + endpoint + " is closed");
  for (uint64_t i = 0; i < total; ++i) {
    Packet pk;
    pk.keep = keep;
    pk.data = data + i * max_packet_;
    pk.len = std::min<uint64_t>(max_packet_, n - i * max_packet_);
    PacketHeader h;
    h.little_endian = host_is_little_endian() ? 1 : 0;
    h.packet_length = pk.len;
    h.msg_length = n;
    h.msg_serial_id = id;
    h.packet_offset = static_cast<uint32_t>(i);
    h.total_packets = static_cast<uint32_t>(total);
    ByteWriter w;
    write_packet_header(w, h);
    pk.header = std::move(w.buf);
    bytes_sent_ += pk.header.size() + pk.len;
    // a message that fits one packet always takes the peer's first socket, so that short control messages reach
    // the peer in the order they were sent; the packets of larger messages are spread over all sockets
    auto& c = total == 1 ? live[0] : live[peer->next++ % live.size()];
    {
      std::lock_guard<std::mutex> q(c->mu);
      c->out.push_back(std::move(pk));
    }
    c->cv.notify_all();  // the writer, and possibly a flush() waiting on the same condition
  }
  ++messages_sent_;
}

void TcpCommunicator::write_loop(std::shared_ptr<Conn> c) {
  for (;;) {
    Packet pk;
    {
      std::unique_lock<std::mutex> l(c->mu);
      c->writing = false;
      c->cv.notify_all();
      c->cv.wait(l, [&] { return !c->out.empty() || c->closed || stopping_; });
      if (c->out.empty()) return;
      pk = std::move(c->out.front());
      c->out.pop_front();
      c->writing = true;
    }
    if (!write_exact(c->fd, pk.header.data(), pk.header.size()) ||
        (pk.len && !write_exact(c->fd, pk.data, pk.len))) {
      c->closed = true;
      std::lock_guard<std::mutex> l(c->mu);
      c->out.clear();
      c->writing = false;
      c->cv.notify_all();
      return;
    }
  }
}

void TcpCommunicator::read_loop(std::shared_ptr<Conn> c) {
  char hdr[PacketHeader::kSize];
  std::string scratch;
  for (;;) {
    if (!read_exact(c->fd, hdr, PacketHeader::kSize)) break;
    PacketHeader h;
    char* dst = nullptr;
    bool dup = false;
    try {
      h = read_packet_header(hdr, PacketHeader::kSize);
      if (h.packet_length > max_packet_ + (1ull << 20)) break;  // not a packet of this protocol
      if (h.msg_length > max_message_) break;                    // larger than this endpoint agrees to buffer
      std::lock_guard<std::mutex> g(c->peer->mu);
      dst = c->peer->agg.reserve(h, &dup);
    } catch (const std::exception&) {
      break;
    }
    if (dup) {  // a repeated packet is read and dropped
      scratch.resize(h.packet_length);
      dst = scratch.empty() ? nullptr : &scratch[0];
    }
    // the payload goes from the socket straight to its place in the message
    if (h.packet_length && !read_exact(c->fd, dst, h.packet_length)) break;
    bytes_received_ += PacketHeader::kSize + h.packet_length;
    std::string msg;
    bool done = false;
    try {
      std::lock_guard<std::mutex> g(c->peer->mu);
      done = c->peer->agg.commit(h, &msg);
    } catch (const std::exception&) {
      break;
    }
    if (done) deliver(c->peer->name, std::move(msg));
  }
  c->closed = true;
  c->cv.notify_all();
}

uint64_t TcpCommunicator::echo(const std::string& stop_message) {
  uint64_t n = 0;
  std::string from, msg;
  while (recv(-1.0, &from, &msg)) {
    if (msg == stop_message) break;
    send(from, std::move(msg));
    msg.clear();
    ++n;
  }
  return n;
}

uint64_t TcpCommunicator::ping_pong(const std::string& endpoint, size_t message_bytes, double seconds, double* elapsed_s) {
  auto payload = std::make_shared<std::string>(message_bytes, '\0');
  const auto t0 = std::chrono::steady_clock::now();
  auto elapsed = [&] { return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count(); };
  uint64_t n = 0;
  std::string from, msg;
  while (elapsed() < seconds) {
    send_view(endpoint, payload->data(), payload->size(), payload);
    if (!recv(60.0, &from, &msg)) throw std::runtime_error("the echo did not come back");
    if (msg.size() != message_bytes) throw std::runtime_error("the echo has the wrong length");
    ++n;
  }
  if (elapsed_s) *elapsed_s = elapsed();
  return n;
}

void TcpCommunicator::deliver(const std::string& from, std::string&& msg) {
  {
    std::lock_guard<std::mutex> g(inbox_mu_);
    inbox_.emplace_back(from, std::move(msg));
  }
  ++messages_received_;
  inbox_cv_.notify_one();
}

bool TcpCommunicator::recv(double timeout_s, std::string* endpoint, std::string* message) {
  std::unique_lock<std::mutex> l(inbox_mu_);
  auto ready = [&] { return !inbox_.empty() || stopping_; };
  if (timeout_s < 0)
    inbox_cv_.wait(l, ready);
  else
    inbox_cv_.wait_for(l, std::chrono::duration<double>(timeout_s), ready);
  if (inbox_.empty()) return false;
  *endpoint = std::move(inbox_.front().first);
  *message = std::move(inbox_.front().second);
  inbox_.pop_front();
  return true;
}

void TcpCommunicator::flush(double timeout_s) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s);
  std::vector<std::shared_ptr<Conn>> conns;
  {
    std::lock_guard<std::mutex> g(peers_mu_);
    conns = all_conns_;
  }
  for (auto& c : conns) {
    std::unique_lock<std::mutex> l(c->mu);
    c->cv.wait_until(l, deadline, [&] { return (c->out.empty() && !c->writing) || c->closed; });
  }
}

void TcpCommunicator::stop() {
  if (stopping_.exchange(true) && listen_fd_ < 0) return;
  if (acceptor_.joinable()) acceptor_.join();
  if (listen_fd_ >= 0) ::close(listen_fd_);
  listen_fd_ = -1;
  std::vector<std::shared_ptr<Conn>> conns;
  {
    std::lock_guard<std::mutex> g(peers_mu_);
    conns.swap(all_conns_);
    peers_.clear();
  }
  for (auto& c : conns) {
    c->closed = true;
    ::shutdown(c->fd, SHUT_RDWR);
    {
      std::lock_guard<std::mutex> l(c->mu);
    }
    c->cv.notify_all();
  }
  for (auto& c : conns) {
    if (c->reader.joinable()) c->reader.join();
    if (c->writer.joinable()) c->writer.join();
    ::close(c->fd);
    c->peer.reset();
  }
  inbox_cv_.notify_all();
}

}  // namespace tnnb
