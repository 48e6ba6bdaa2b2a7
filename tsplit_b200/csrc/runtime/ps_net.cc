// Parameter server over TCP: workers in other processes (or on other hosts) reach the shards of a server process.
//
// The reference's workers and servers are separate processes joined by ps-lite's ZeroMQ van
// (ps-lite/src/van.cc, zmq_van.h; roles from DMLC_ROLE, src/ps/worker.cc:20-60).  Here the shard store is
// csrc/runtime/ps_shards.cc; this file gives it a wire: the server process listens on a port (of the loopback
// interface unless told otherwise) and serves every
// connection from a thread of its own, which turns each request into the in-process call (tsb_ps_init / push / pull /
// barrier / sparse_* / heartbeat) on the shared store.  One connection per worker, requests answered in order.
//
//   request : Header {magic, op, worker, key, n, aux} + payload (floats, or int64 rows then floats for sparse ops)
//   reply   : Reply {status, ts, n} + n floats
//
// A worker that disappears closes its connection: the server thread ends, counts it in `gone`, and (because the
// store's barrier counts arrivals) releases nobody: the others learn of it from tsb_psnet_gone() / a heartbeat query,
// as in the reference, where a dead node is found by the scheduler's heartbeat timeout (ps-lite/src/postoffice.cc).
// Every request of a worker has a timeout on the worker's side, so a silent server (or a barrier that a dead
// worker never joins) ends with an error instead of a hang.
#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

extern "C" {
// the in-process store (ps_shards.cc)
int tsb_ps_init(void* h, int64_t key, const float* data, int64_t len);
int64_t tsb_ps_push(void* h, int worker, int64_t key, const float* data, int64_t len);
int64_t tsb_ps_pull(void* h, int worker, int64_t key, float* out, int64_t len);
int tsb_ps_wait(void* h, int64_t ts);
int tsb_ps_barrier(void* h);
int tsb_ps_release_barrier(void* h);
int tsb_ps_sparse_push(void* h, int worker, int64_t key, const int64_t* rows, int64_t n_rows, const float* data,
                       int64_t cols);
int tsb_ps_sparse_pull(void* h, int64_t key, const int64_t* rows, int64_t n_rows, float* out, int64_t cols);
int tsb_ps_heartbeat(void* h, int node);
int tsb_ps_dead_nodes(void* h, int timeout_ms, int* out, int max_out);
}

namespace {

constexpr uint32_t MAGIC = 0x54535053;   // "TSPS"
enum Op : uint32_t { OP_INIT = 1, OP_PUSH, OP_PULL, OP_BARRIER, OP_SPARSE_PUSH, OP_SPARSE_PULL, OP_HEARTBEAT, OP_DEAD, OP_BYE };

struct Header {
  uint32_t magic, op;
  int32_t worker, pad;
  int64_t key, n, aux;
};
struct Reply {
  int32_t status, pad;
  int64_t ts, n;
};

bool send_all(int fd, const void* p, size_t n) {
  const char* c = static_cast<const char*>(p);
  while (n) {
    const ssize_t k = ::send(fd, c, n, MSG_NOSIGNAL);
    if (k <= 0) return false;
    c += k; n -= (size_t)k;
  }
  return true;
}
bool recv_all(int fd, void* p, size_t n) {
  char* c = static_cast<char*>(p);
  while (n) {
    const ssize_t k = ::recv(fd, c, n, 0);
    if (k <= 0) return false;
    c += k; n -= (size_t)k;
  }
  return true;
}
void set_timeouts(int fd, int ms) {
  timeval tv;
  tv.tv_sec = ms / 1000; tv.tv_usec = (ms % 1000) * 1000;
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
}

struct Server {
  void* store = nullptr;
  int listen_fd = -1, port = 0;
  std::atomic<bool> stop{false};
  std::atomic<int> connected{0}, gone{0}, accepted{0};
  std::thread acceptor;
  std::mutex mu;
  std::vector<std::thread> conns;
  std::vector<int> fds;
};

void serve_connection(Server* s, int fd) {
  std::vector<float> buf;
  std::vector<int64_t> rows;
  bool said_bye = false;
  for (;;) {
    Header h;
    if (!recv_all(fd, &h, sizeof h)) break;        // the peer closed, or tsb_psnet_stop shut the socket down
    if (h.magic != MAGIC || h.n < 0 || h.n > (int64_t(1) << 33)) break;
    Reply r{0, 0, 0, 0};
    bool ok = true;
    switch (h.op) {
      case OP_INIT:
        buf.resize((size_t)(h.aux ? h.n : 0));
        if (h.aux) ok = recv_all(fd, buf.data(), (size_t)h.n * 4);
        if (ok) r.status = tsb_ps_init(s->store, h.key, h.aux ? buf.data() : nullptr, h.n);
        break;
      case OP_PUSH:
        buf.resize((size_t)h.n);
        ok = recv_all(fd, buf.data(), (size_t)h.n * 4);
        if (ok) {
          r.ts = tsb_ps_push(s->store, h.worker, h.key, buf.data(), h.n);
          if (r.ts > 0) tsb_ps_wait(s->store, r.ts); else r.status = 1;
        }
        break;
      case OP_PULL:
        buf.resize((size_t)h.n);
        r.ts = tsb_ps_pull(s->store, h.worker, h.key, buf.data(), h.n);
        if (r.ts > 0) { tsb_ps_wait(s->store, r.ts); r.n = h.n; } else r.status = 1;
        break;
      case OP_BARRIER:
        // a barrier that a departed worker can never join is answered at once
        r.status = s->gone.load() > 0 ? 5 : tsb_ps_barrier(s->store);
        break;
      case OP_SPARSE_PUSH:            // n rows, aux columns: rows then values
        rows.resize((size_t)h.n);
        buf.resize((size_t)(h.n * h.aux));
        ok = recv_all(fd, rows.data(), (size_t)h.n * 8) && recv_all(fd, buf.data(), buf.size() * 4);
        if (ok) r.status = tsb_ps_sparse_push(s->store, h.worker, h.key, rows.data(), h.n, buf.data(), h.aux);
        break;
      case OP_SPARSE_PULL:
        rows.resize((size_t)h.n);
        buf.resize((size_t)(h.n * h.aux));
        ok = recv_all(fd, rows.data(), (size_t)h.n * 8);
        if (ok) {
          r.status = tsb_ps_sparse_pull(s->store, h.key, rows.data(), h.n, buf.data(), h.aux);
          if (r.status == 0) r.n = h.n * h.aux;
        }
        break;
      case OP_HEARTBEAT:
        r.status = tsb_ps_heartbeat(s->store, h.worker);
        break;
      case OP_DEAD: {                 // aux = timeout in ms; reply: node ids as floats
        int ids[64];
        const int k = tsb_ps_dead_nodes(s->store, (int)h.aux, ids, 64);
        buf.resize((size_t)(k > 0 ? k : 0));
        for (int i = 0; i < k; ++i) buf[(size_t)i] = (float)ids[i];
        r.n = k > 0 ? k : 0;
        break;
      }
      case OP_BYE:
        said_bye = true;
        break;
      default:
        r.status = 2;
    }
    if (!ok) break;
    if (!send_all(fd, &r, sizeof r)) break;
    if (r.n > 0 && !send_all(fd, buf.data(), (size_t)r.n * 4)) break;
    if (said_bye) break;
  }
  ::close(fd);
  if (!said_bye && !s->stop.load()) {
    s->gone.fetch_add(1);
    tsb_ps_release_barrier(s->store);          // whoever waits for this worker in a barrier gets status 5
  }
  s->connected.fetch_sub(1);
}

void accept_loop(Server* s) {
  while (!s->stop.load()) {
    sockaddr_in peer;
    socklen_t len = sizeof peer;
    const int fd = ::accept(s->listen_fd, reinterpret_cast<sockaddr*>(&peer), &len);
    if (fd < 0) continue;                      // the listening socket has a receive timeout
    set_timeouts(fd, 0);                       // a served connection waits for its worker's next request
    s->connected.fetch_add(1);
    s->accepted.fetch_add(1);
    std::lock_guard<std::mutex> g(s->mu);
    s->fds.push_back(fd);
    s->conns.emplace_back(serve_connection, s, fd);
  }
}

struct Client {
  int fd = -1;
  int timeout_ms = 30000;
};

}  // namespace

extern "C" {

// Serve `store` (a tsb_ps_create handle) on `port` (0 = pick one) of the interface with address `bind_addr`
// (dotted quad; null or empty = 127.0.0.1, the loopback interface: the requests carry no authentication, so the
// listener is reachable from this machine only unless the caller names another interface).  Returns a handle or null.
void* tsb_psnet_serve(void* store, int port, const char* bind_addr) {
  if (!store) return nullptr;
  in_addr where;
  where.s_addr = htonl(INADDR_LOOPBACK);
  if (bind_addr && bind_addr[0] && inet_pton(AF_INET, bind_addr, &where) != 1) return nullptr;
  const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return nullptr;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in addr;
  std::memset(&addr, 0, sizeof addr);
  addr.sin_family = AF_INET;
  addr.sin_addr = where;
  addr.sin_port = htons((uint16_t)port);
  if (::bind(fd, reinterpret_cast<sockaddr*>(&addr), sizeof addr) != 0 || ::listen(fd, 64) != 0) {
    ::close(fd);
    return nullptr;
  }
  socklen_t len = sizeof addr;
  getsockname(fd, reinterpret_cast<sockaddr*>(&addr), &len);
  timeval tv{0, 200000};                       // accept() wakes up five times a second to see `stop`
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  Server* s = new Server();
  s->store = store; s->listen_fd = fd; s->port = ntohs(addr.sin_port);
  s->acceptor = std::thread(accept_loop, s);
  return s;
}

int tsb_psnet_port(void* server) { return server ? static_cast<Server*>(server)->port : 0; }
// connections accepted since the listener started
int tsb_psnet_accepted(void* server) { return server ? static_cast<Server*>(server)->accepted.load() : 0; }
int tsb_psnet_connected(void* server) { return server ? static_cast<Server*>(server)->connected.load() : 0; }
// workers whose connection ended without a goodbye
int tsb_psnet_gone(void* server) { return server ? static_cast<Server*>(server)->gone.load() : 0; }

void tsb_psnet_stop(void* server) {
  Server* s = static_cast<Server*>(server);
  if (!s) return;
  s->stop.store(true);
  if (s->acceptor.joinable()) s->acceptor.join();
  ::close(s->listen_fd);
  tsb_ps_release_barrier(s->store);            // connection threads blocked in a barrier come back
  {
    std::lock_guard<std::mutex> g(s->mu);
    for (int fd : s->fds) ::shutdown(fd, SHUT_RDWR);
  }
  for (auto& t : s->conns)
    if (t.joinable()) t.join();
  delete s;
}

// Worker side.  Returns a handle or null (no server within timeout_ms).
void* tsb_psnet_connect(const char* host, int port, int timeout_ms) {
  addrinfo hints, *res = nullptr;
  std::memset(&hints, 0, sizeof hints);
  hints.ai_family = AF_INET; hints.ai_socktype = SOCK_STREAM;
  char portstr[16];
  snprintf(portstr, sizeof portstr, "%d", port);
  if (getaddrinfo(host, portstr, &hints, &res) != 0 || !res) return nullptr;
  int fd = -1;
  const int tries = timeout_ms / 50 + 1;
  for (int t = 0; t < tries && fd < 0; ++t) {
    fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd >= 0 && ::connect(fd, res->ai_addr, res->ai_addrlen) != 0) { ::close(fd); fd = -1; usleep(50000); }
  }
  freeaddrinfo(res);
  if (fd < 0) return nullptr;
  Client* c = new Client();
  c->fd = fd; c->timeout_ms = timeout_ms > 0 ? timeout_ms : 30000;
  set_timeouts(fd, c->timeout_ms);
  return c;
}

// One request / reply.  in_rows (int64, n of them) only for the sparse ops; in_data: in_n floats; the reply's floats
// go to out (room for out_cap).  Returns 0, the server's status, or -1 for a broken / timed-out connection.
int tsb_psnet_request(void* client, int op, int worker, int64_t key, int64_t n, int64_t aux, const int64_t* in_rows,
                      const float* in_data, int64_t in_n, float* out, int64_t out_cap, int64_t* ts_out,
                      int64_t* out_n) {
  Client* c = static_cast<Client*>(client);
  if (!c || c->fd < 0) return -1;
  Header h{MAGIC, (uint32_t)op, worker, 0, key, n, aux};
  if (!send_all(c->fd, &h, sizeof h)) return -1;
  if (in_rows && !send_all(c->fd, in_rows, (size_t)n * 8)) return -1;
  if (in_data && in_n > 0 && !send_all(c->fd, in_data, (size_t)in_n * 4)) return -1;
  Reply r;
  if (!recv_all(c->fd, &r, sizeof r)) return -1;
  if (ts_out) *ts_out = r.ts;
  if (out_n) *out_n = r.n;
  if (r.n > 0) {
    if (r.n > out_cap || !out) {               // drain what cannot be stored, then report
      std::vector<float> sink((size_t)r.n);
      recv_all(c->fd, sink.data(), (size_t)r.n * 4);
      return -1;
    }
    if (!recv_all(c->fd, out, (size_t)r.n * 4)) return -1;
  }
  return r.status;
}

void tsb_psnet_close(void* client, int say_bye) {
  Client* c = static_cast<Client*>(client);
  if (!c) return;
  if (c->fd >= 0) {
    if (say_bye) {
      Header h{MAGIC, OP_BYE, 0, 0, 0, 0, 0};
      Reply r;
      if (send_all(c->fd, &h, sizeof h)) recv_all(c->fd, &r, sizeof r);
    }
    ::close(c->fd);
  }
  delete c;
}

}  // extern "C"
