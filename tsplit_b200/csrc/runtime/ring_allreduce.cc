// Host ring all-reduce over TCP sockets: reduce-scatter, all-gather, optional
// average.  Each rank listens on base_port + rank and connects to its right
// neighbour; the vector is cut into `n` segments (remainder spread over the first
// ones), and 2(n-1) steps move one segment per step around the ring.
//
// Capability parity: the reference's ZeroMQ ring (src/communication/
// c_communication_nthread.cc:39-125,218-246,372-398,478-496: REQ/REP pairs with
// "ok" acknowledgements, per-worker segments, divide by n at the end).  Plain
// POSIX sockets replace ZeroMQ; sends and receives of a step run on two threads
// so a step never deadlocks on socket buffers.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

struct Ring {
  int n, id;
  int listen_fd = -1, left_fd = -1, right_fd = -1;   // receive from left, send to right
  std::vector<float> recv_buf;
};

bool send_all(int fd, const void* buf, size_t len) {
  const char* p = static_cast<const char*>(buf);
  while (len) {
    ssize_t k = ::send(fd, p, len, MSG_NOSIGNAL);
    if (k <= 0) return false;
    p += k; len -= (size_t)k;
  }
  return true;
}
bool recv_all(int fd, void* buf, size_t len) {
  char* p = static_cast<char*>(buf);
  while (len) {
    ssize_t k = ::recv(fd, p, len, 0);
    if (k <= 0) return false;
    p += k; len -= (size_t)k;
  }
  return true;
}

void seg_bounds(int64_t len, int n, int s, int64_t* b, int64_t* e) {
  const int64_t base = len / n, rem = len % n;
  *b = s * base + (s < rem ? s : rem);
  *e = *b + base + (s < rem ? 1 : 0);
}

}  // namespace

extern "C" {

// Bind + connect.  timeout_ms bounds the wait for the neighbour.  Returns a handle or null.
void* tsb_ring_connect(int n, int id, const char* host, int base_port, int timeout_ms) {
  if (n < 1 || id < 0 || id >= n) return nullptr;
  Ring* r = new Ring();
  r->n = n; r->id = id;
  if (n == 1) return r;
  r->listen_fd = ::socket(AF_INET, SOCK_STREAM, 0);
  int one = 1;
  ::setsockopt(r->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  // every rank of this ring lives at `host` (default: the loopback interface), so that is where this rank listens
  ::inet_pton(AF_INET, host && *host ? host : "127.0.0.1", &addr.sin_addr);
  addr.sin_port = htons((uint16_t)(base_port + id));
  if (::bind(r->listen_fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(r->listen_fd, 4) != 0) {
    ::close(r->listen_fd);
    delete r;
    return nullptr;
  }
  // connect to the right neighbour (retry until it listens), then accept the left one
  const int right = (id + 1) % n;
  sockaddr_in peer{};
  peer.sin_family = AF_INET;
  peer.sin_port = htons((uint16_t)(base_port + right));
  ::inet_pton(AF_INET, host && *host ? host : "127.0.0.1", &peer.sin_addr);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms > 0 ? timeout_ms : 10000);
  for (;;) {
    r->right_fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (::connect(r->right_fd, reinterpret_cast<sockaddr*>(&peer), sizeof(peer)) == 0) break;
    ::close(r->right_fd);
    r->right_fd = -1;
    if (std::chrono::steady_clock::now() > deadline) {
      ::close(r->listen_fd);
      delete r;
      return nullptr;
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
  ::setsockopt(r->right_fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  timeval tv{};
  tv.tv_sec = (timeout_ms > 0 ? timeout_ms : 10000) / 1000 + 1;
  ::setsockopt(r->listen_fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  r->left_fd = ::accept(r->listen_fd, nullptr, nullptr);
  if (r->left_fd < 0) {
    ::close(r->right_fd); ::close(r->listen_fd);
    delete r;
    return nullptr;
  }
  ::setsockopt(r->left_fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));   // a dead neighbour ends the wait
  return r;
}

// In-place sum (average != 0: mean) of `data` over all ranks.  0 = ok, 4 = a neighbour went away.
int tsb_ring_allreduce(void* h, float* data, int64_t len, int average) {
  Ring* r = static_cast<Ring*>(h);
  if (!r || len < 0) return 1;
  const int n = r->n, id = r->id;
  if (n > 1) {
    int64_t maxseg = len / n + 1;
    r->recv_buf.resize((size_t)maxseg);
    bool ok = true;
    for (int step = 0; step < 2 * (n - 1) && ok; ++step) {
      const bool reduce = step < n - 1;
      const int s_send = reduce ? (id - step + n) % n : (id + 1 - (step - (n - 1)) + n) % n;
      const int s_recv = (s_send - 1 + n) % n;
      int64_t sb, se, rb, re;
      seg_bounds(len, n, s_send, &sb, &se);
      seg_bounds(len, n, s_recv, &rb, &re);
      bool sent_ok = true;
      std::thread tx([&] { sent_ok = send_all(r->right_fd, data + sb, sizeof(float) * (size_t)(se - sb)); });
      float* dst = reduce ? r->recv_buf.data() : data + rb;
      const bool recv_ok = recv_all(r->left_fd, dst, sizeof(float) * (size_t)(re - rb));
      tx.join();
      ok = sent_ok && recv_ok;
      if (ok && reduce)
        for (int64_t i = 0; i < re - rb; ++i) data[rb + i] += r->recv_buf[(size_t)i];
    }
    if (!ok) return 4;
  }
  if (average && n > 1) {
    const float inv = 1.f / (float)n;
    for (int64_t i = 0; i < len; ++i) data[i] *= inv;
  }
  return 0;
}

void tsb_ring_close(void* h) {
  Ring* r = static_cast<Ring*>(h);
  if (!r) return;
  if (r->left_fd >= 0) ::close(r->left_fd);
  if (r->right_fd >= 0) ::close(r->right_fd);
  if (r->listen_fd >= 0) ::close(r->listen_fd);
  delete r;
}

}  // extern "C"
