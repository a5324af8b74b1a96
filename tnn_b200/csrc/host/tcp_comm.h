// TCP transport for wire-format messages between hosts (the multi-node control and data plane of the
// coordinator / worker protocol; inside one NVSwitch box tensors move over NCCL or peer memory instead).
//
// Behaviour follows the reference's TCP communicator (include/distributed/tcp_communicator.hpp:106-120
// server start, :208-218 and :283-302 identity handshake, include/distributed/chunking.hpp:46-71 slicing):
//   * every endpoint listens on one port and is named "ip:port" after it;
//   * connect() opens `sockets_per_endpoint` TCP_NODELAY sockets to a peer and sends, on each, this side's
//     listening port as a little-endian i32, so that the acceptor can name the peer;
//   * send() cuts a message into packets of at most `max_packet_size` payload bytes, each behind the 36-byte
//     PacketHeader, and spreads the packets over the peer's sockets; the receiver reassembles them in any order.
//     Messages of a single packet all use the first socket and therefore arrive in order.
// The implementation is plain POSIX sockets with one reader and one writer thread per socket (the reference uses
// asio coroutines on a pool of I/O threads); send() only queues, so compute overlaps with the transfer.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "wire.h"

namespace tnnb {

class TcpCommunicator {
 public:
  // `bind_host` is the address to listen on and the ip of this endpoint's name; port 0 asks for a free port.
  TcpCommunicator(std::string bind_host, int port, int sockets_per_endpoint = 4, uint64_t max_packet_size = 4ull << 20);
  ~TcpCommunicator();
  TcpCommunicator(const TcpCommunicator&) = delete;
  TcpCommunicator& operator=(const TcpCommunicator&) = delete;

  int start();                                         // bind + listen + accept thread; returns the listening port
  std::string endpoint() const;                        // "ip:port" of this side
  std::string connect(const std::string& host, int port, double timeout_s = 10.0);  // returns the peer's endpoint name
  bool connected(const std::string& endpoint);
  void send(const std::string& endpoint, std::string message);  // queues; throws if the peer is unknown or closed
  // The same without a copy: `data` must stay valid until `keep` (any owner of it) is released, which happens on a
  // writer thread once the last packet has been written.
  void send_view(const std::string& endpoint, const char* data, size_t n, std::shared_ptr<const void> keep);
  // Next complete message, oldest first. False when `timeout_s` ran out (negative = wait for ever) or after stop().
  bool recv(double timeout_s, std::string* endpoint, std::string* message);
  // Benchmark loops that stay inside the communicator (the reference's tcp_communicator_benchmark.cpp bounces
  // messages between two of its communicators without leaving C++ either):
  //   echo()       send every received message back to its sender (the received buffer itself, no copy) until a
  //                message equal to `stop_message` arrives or the endpoint stops; returns the number echoed.
  //   ping_pong()  send one `message_bytes` message to `endpoint` and wait for the echo, again and again for
  //                `seconds`; returns the number of round trips and stores the elapsed time. The same buffer is
  //                sent every time, so no copy is made on this side either.
  uint64_t echo(const std::string& stop_message);
  uint64_t ping_pong(const std::string& endpoint, size_t message_bytes, double seconds, double* elapsed_s);
  void flush(double timeout_s = 30.0);                 // wait until every queued packet has been written
  void stop();

  // Longest message (bytes) this endpoint lets a peer announce; default 16 GiB.
  void set_max_message_bytes(uint64_t n) { max_message_ = n; }
  uint64_t bytes_sent() const { return bytes_sent_; }
  uint64_t bytes_received() const { return bytes_received_; }
  uint64_t messages_sent() const { return messages_sent_; }
  uint64_t messages_received() const { return messages_received_; }
  std::vector<std::string> peers();

 private:
  struct Peer;
  struct Packet {  // header bytes + a view into the message they belong to (no per-packet copy of the payload)
    std::string header;
    std::shared_ptr<const void> keep;  // owner of the message bytes
    const char* data = nullptr;        // this packet's payload inside them
    size_t len = 0;
  };
  struct Conn {
    int fd = -1;
    std::shared_ptr<Peer> peer;
    std::thread reader, writer;
    std::mutex mu;
    std::condition_variable cv;
    std::deque<Packet> out;  // packets waiting to be written
    bool writing = false;
    std::atomic<bool> closed{false};
  };
  struct Peer {
    std::string name;
    std::mutex mu;  // guards conns, next, agg
    std::vector<std::shared_ptr<Conn>> conns;
    size_t next = 0;
    Aggregator agg;
  };

  std::shared_ptr<Peer> peer_for(const std::string& name, bool create);
  void adopt(int fd, const std::string& peer_name);
  void accept_loop();
  void read_loop(std::shared_ptr<Conn> c);
  void write_loop(std::shared_ptr<Conn> c);
  void deliver(const std::string& from, std::string&& msg);

  std::string host_;
  int port_;
  int sockets_;
  uint64_t max_packet_;
  std::atomic<uint64_t> max_message_{16ull << 30};  // a header that announces a longer message closes its connection
  int listen_fd_ = -1;
  std::thread acceptor_;
  std::atomic<bool> stopping_{false};
  std::atomic<uint64_t> next_msg_id_{1}, bytes_sent_{0}, bytes_received_{0}, messages_sent_{0}, messages_received_{0};

  std::mutex peers_mu_;
  std::map<std::string, std::shared_ptr<Peer>> peers_;
  std::vector<std::shared_ptr<Conn>> all_conns_;  // under peers_mu_

  std::mutex inbox_mu_;
  std::condition_variable inbox_cv_;
  std::deque<std::pair<std::string, std::string>> inbox_;
};

}  // namespace tnnb
