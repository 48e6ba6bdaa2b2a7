// Parameter-server shards: key -> dense vector stores partitioned over S server
// shards, a 5-thread request pool per agent, timestamps to wait on, BSP barrier,
// server-side PS functions, heartbeats, and an at-least-once delivery layer with
// sequence-number de-duplication (resend on a dropped message; drop rate is a
// fault-injection knob).
//
// Capability parity: the vendored ps-lite of the reference — PSF functions
// (ps-lite/include/ps/psf/PSFunc.h:4-22, PSFHandle.h:53-280), PSAgent's even split
// of a tensor over the servers and its thread pool (psmodel/PSAgent.h:33-81,
// 245-322), worker BSP/ASP entry points (src/ps/worker.cc:108-133), heartbeat /
// dead-node detection (van.cc:574-587, postoffice.cc:198-216), Resender
// (resender.h:15-129) and PS_DROP_MSG (van.cc:420-426).  Everything is host code
// in one process (server shards are threads); on GPUs the same push/pull
// contract is served by the fused all-reduce kernel with shard = owning rank.
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <mutex>
#include <queue>
#include <random>
#include <set>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

using Clock = std::chrono::steady_clock;

struct Shard {
  std::mutex mu;
  std::unordered_map<int64_t, std::vector<float>> store;   // key -> this shard's slice
  std::set<std::pair<int, int64_t>> seen;                  // (worker, seq) already applied
};

struct PS {
  int num_servers, num_workers;
  int drop_percent, resend_ms;
  std::vector<Shard> shards;
  std::unordered_map<int64_t, int64_t> lengths;            // key -> full length
  std::mutex meta_mu;

  // request pool
  std::vector<std::thread> pool;
  std::queue<std::pair<int64_t, std::function<void()>>> tasks;
  std::mutex task_mu;
  std::condition_variable task_cv, done_cv;
  std::set<int64_t> outstanding;
  int64_t next_ts = 1;
  bool stop = false;

  // barrier
  std::mutex bar_mu;
  std::condition_variable bar_cv;
  int bar_count = 0;
  int64_t bar_gen = 0;
  int64_t bar_broken = 0;      // bumped by tsb_ps_release_barrier

  // heartbeats
  std::mutex hb_mu;
  std::map<int, Clock::time_point> last_seen;

  // delivery statistics
  std::atomic<int64_t> sent{0}, dropped{0}, resent{0}, duplicates{0};
  std::atomic<int64_t> seq{1};
  std::mt19937 rng{12345};
  std::mutex rng_mu;

  PS(int s, int w, int drop, int resend) : num_servers(s), num_workers(w), drop_percent(drop), resend_ms(resend),
                                           shards(s) {
    for (int i = 0; i < 5; ++i) pool.emplace_back([this] { work(); });
  }
  ~PS() {
    {
      std::lock_guard<std::mutex> g(task_mu);
      stop = true;
    }
    task_cv.notify_all();
    for (auto& t : pool) t.join();
  }

  void work() {
    for (;;) {
      std::pair<int64_t, std::function<void()>> job;
      {
        std::unique_lock<std::mutex> lk(task_mu);
        task_cv.wait(lk, [this] { return stop || !tasks.empty(); });
        if (stop && tasks.empty()) return;
        job = std::move(tasks.front());
        tasks.pop();
      }
      job.second();
      {
        std::lock_guard<std::mutex> g(task_mu);
        outstanding.erase(job.first);
      }
      done_cv.notify_all();
    }
  }

  int64_t submit(std::function<void()> fn) {
    std::lock_guard<std::mutex> g(task_mu);
    const int64_t ts = next_ts++;
    outstanding.insert(ts);
    tasks.push({ts, std::move(fn)});
    task_cv.notify_one();
    return ts;
  }

  void wait(int64_t ts) {
    std::unique_lock<std::mutex> lk(task_mu);
    done_cv.wait(lk, [&] { return outstanding.count(ts) == 0; });
  }

  bool lose_message() {
    if (drop_percent <= 0) return false;
    std::lock_guard<std::mutex> g(rng_mu);
    return (int)(rng() % 100) < drop_percent;
  }

  // slice [begin, end) of a length-n vector owned by shard s
  void slice(int64_t n, int s, int64_t* b, int64_t* e) const {
    const int64_t per = (n + num_servers - 1) / num_servers;
    *b = std::min<int64_t>(n, per * s);
    *e = std::min<int64_t>(n, per * (s + 1));
  }

  // At-least-once delivery of one request to one shard: a lost request (or a lost
  // acknowledgement) is re-sent with the same sequence number after resend_ms, up to
  // 10 times; the shard applies each (worker, seq) once.
  bool deliver(int s, int worker, const std::function<void(Shard&)>& apply) {
    const int64_t my_seq = seq++;
    for (int attempt = 0; attempt <= 10; ++attempt) {
      ++sent;
      if (attempt) ++resent;
      if (lose_message()) {            // request lost on the way
        ++dropped;
        std::this_thread::sleep_for(std::chrono::milliseconds(resend_ms));
        continue;
      }
      Shard& sh = shards[s];
      {
        std::lock_guard<std::mutex> g(sh.mu);
        if (sh.seen.insert({worker, my_seq}).second) apply(sh);
        else ++duplicates;
      }
      if (lose_message()) {            // acknowledgement lost: the sender will re-send
        ++dropped;
        std::this_thread::sleep_for(std::chrono::milliseconds(resend_ms));
        continue;
      }
      return true;
    }
    return false;
  }
};

int64_t key_len(PS* p, int64_t key) {
  std::lock_guard<std::mutex> g(p->meta_mu);
  auto it = p->lengths.find(key);
  return it == p->lengths.end() ? -1 : it->second;
}

}  // namespace

extern "C" {

void* tsb_ps_create(int num_servers, int num_workers, int drop_percent, int resend_timeout_ms) {
  if (num_servers < 1 || num_workers < 1) return nullptr;
  return new PS(num_servers, num_workers, drop_percent, resend_timeout_ms > 0 ? resend_timeout_ms : 1);
}
void tsb_ps_destroy(void* h) { delete static_cast<PS*>(h); }

// Create key with `len` floats: copies `data`, or zeros when data == null (InitAllZeros).
int tsb_ps_init(void* h, int64_t key, const float* data, int64_t len) {
  PS* p = static_cast<PS*>(h);
  if (!p || len <= 0) return 1;
  {
    std::lock_guard<std::mutex> g(p->meta_mu);
    p->lengths[key] = len;
  }
  for (int s = 0; s < p->num_servers; ++s) {
    int64_t b, e;
    p->slice(len, s, &b, &e);
    std::lock_guard<std::mutex> g(p->shards[s].mu);
    auto& v = p->shards[s].store[key];
    v.assign(e - b, 0.f);
    if (data) std::memcpy(v.data(), data + b, sizeof(float) * (e - b));
  }
  return 0;
}

// DensePush: server += data.  Asynchronous; returns a timestamp (> 0) to wait on, or -1.
int64_t tsb_ps_push(void* h, int worker, int64_t key, const float* data, int64_t len) {
  PS* p = static_cast<PS*>(h);
  if (!p || key_len(p, key) != len) return -1;
  return p->submit([=] {
    for (int s = 0; s < p->num_servers; ++s) {
      int64_t b, e;
      p->slice(len, s, &b, &e);
      if (e > b) p->deliver(s, worker, [&](Shard& sh) {
        auto& v = sh.store[key];
        for (int64_t i = 0; i < e - b; ++i) v[i] += data[b + i];
      });
    }
  });
}

// DensePull: out = server.
int64_t tsb_ps_pull(void* h, int worker, int64_t key, float* out, int64_t len) {
  PS* p = static_cast<PS*>(h);
  if (!p || key_len(p, key) != len) return -1;
  return p->submit([=] {
    for (int s = 0; s < p->num_servers; ++s) {
      int64_t b, e;
      p->slice(len, s, &b, &e);
      if (e > b) {
        Shard& sh = p->shards[s];
        std::lock_guard<std::mutex> g(sh.mu);
        std::memcpy(out + b, sh.store[key].data(), sizeof(float) * (e - b));
      }
    }
  });
}

int tsb_ps_wait(void* h, int64_t ts) {
  PS* p = static_cast<PS*>(h);
  if (!p || ts <= 0) return 1;
  p->wait(ts);
  return 0;
}

// Blocks until num_workers callers have arrived (Postoffice::Barrier among workers).  Returns 0, or 5 when the
// barrier was released by tsb_ps_release_barrier instead (a worker is known to be gone, or the server shuts down).
int tsb_ps_barrier(void* h) {
  PS* p = static_cast<PS*>(h);
  std::unique_lock<std::mutex> lk(p->bar_mu);
  const int64_t gen = p->bar_gen;
  const int64_t broken = p->bar_broken;
  if (++p->bar_count == p->num_workers) {
    p->bar_count = 0;
    ++p->bar_gen;
    p->bar_cv.notify_all();
  } else {
    p->bar_cv.wait(lk, [&] { return p->bar_gen != gen || p->bar_broken != broken; });
    if (p->bar_gen == gen) return 5;           // released without everybody
  }
  return 0;
}

// Release every caller that waits in the barrier now, with status 5, and forget their arrivals.
int tsb_ps_release_barrier(void* h) {
  PS* p = static_cast<PS*>(h);
  if (!p) return 1;
  std::lock_guard<std::mutex> lk(p->bar_mu);
  p->bar_count = 0;
  ++p->bar_broken;
  p->bar_cv.notify_all();
  return 0;
}

// Row-sparse push / pull on a [rows, cols] matrix stored row-major under `key`.
int tsb_ps_sparse_push(void* h, int worker, int64_t key, const int64_t* rows, int64_t n_rows, const float* data,
                       int64_t cols) {
  PS* p = static_cast<PS*>(h);
  const int64_t len = key_len(p, key);
  if (len < 0 || cols <= 0) return 1;
  for (int64_t r = 0; r < n_rows; ++r) {
    const int64_t off = rows[r] * cols;
    if (off < 0 || off + cols > len) return 1;
    for (int s = 0; s < p->num_servers; ++s) {
      int64_t b, e;
      p->slice(len, s, &b, &e);
      const int64_t lo = std::max(off, b), hi = std::min(off + cols, e);
      if (hi > lo) p->deliver(s, worker, [&](Shard& sh) {
        auto& v = sh.store[key];
        for (int64_t i = lo; i < hi; ++i) v[i - b] += data[r * cols + (i - off)];
      });
    }
  }
  return 0;
}
int tsb_ps_sparse_pull(void* h, int64_t key, const int64_t* rows, int64_t n_rows, float* out, int64_t cols) {
  PS* p = static_cast<PS*>(h);
  const int64_t len = key_len(p, key);
  if (len < 0 || cols <= 0) return 1;
  for (int64_t r = 0; r < n_rows; ++r) {
    const int64_t off = rows[r] * cols;
    if (off < 0 || off + cols > len) return 1;
    for (int s = 0; s < p->num_servers; ++s) {
      int64_t b, e;
      p->slice(len, s, &b, &e);
      const int64_t lo = std::max(off, b), hi = std::min(off + cols, e);
      if (hi > lo) {
        std::lock_guard<std::mutex> g(p->shards[s].mu);
        const auto& v = p->shards[s].store[key];
        for (int64_t i = lo; i < hi; ++i) out[r * cols + (i - off)] = v[i - b];
      }
    }
  }
  return 0;
}

// Column range [c0, c1) of a [rows, cols] matrix (PSMatrix pushCols / pullCols).
int tsb_ps_cols(void* h, int worker, int64_t key, int64_t rows, int64_t cols, int64_t c0, int64_t c1, float* data,
                int push) {
  PS* p = static_cast<PS*>(h);
  const int64_t len = key_len(p, key);
  if (len != rows * cols || c0 < 0 || c1 > cols || c0 >= c1) return 1;
  const int64_t w = c1 - c0;
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t off = r * cols + c0;
    for (int s = 0; s < p->num_servers; ++s) {
      int64_t b, e;
      p->slice(len, s, &b, &e);
      const int64_t lo = std::max(off, b), hi = std::min(off + w, e);
      if (hi <= lo) continue;
      if (push) {
        p->deliver(s, worker, [&](Shard& sh) {
          auto& v = sh.store[key];
          for (int64_t i = lo; i < hi; ++i) v[i - b] += data[r * w + (i - off)];
        });
      } else {
        std::lock_guard<std::mutex> g(p->shards[s].mu);
        const auto& v = p->shards[s].store[key];
        for (int64_t i = lo; i < hi; ++i) data[r * w + (i - off)] = v[i - b];
      }
    }
  }
  return 0;
}

// Server-side functions evaluated shard by shard.
double tsb_ps_norm2(void* h, int64_t key) {
  PS* p = static_cast<PS*>(h);
  double acc = 0;
  for (auto& sh : p->shards) {
    std::lock_guard<std::mutex> g(sh.mu);
    auto it = sh.store.find(key);
    if (it != sh.store.end()) for (float v : it->second) acc += (double)v * v;
  }
  return std::sqrt(acc);
}
int64_t tsb_ps_nnz(void* h, int64_t key) {
  PS* p = static_cast<PS*>(h);
  int64_t n = 0;
  for (auto& sh : p->shards) {
    std::lock_guard<std::mutex> g(sh.mu);
    auto it = sh.store.find(key);
    if (it != sh.store.end()) for (float v : it->second) n += (v != 0.f);
  }
  return n;
}
double tsb_ps_dot(void* h, int64_t k1, int64_t k2) {
  PS* p = static_cast<PS*>(h);
  double acc = 0;
  for (auto& sh : p->shards) {
    std::lock_guard<std::mutex> g(sh.mu);
    auto a = sh.store.find(k1), b = sh.store.find(k2);
    if (a == sh.store.end() || b == sh.store.end() || a->second.size() != b->second.size()) continue;
    for (size_t i = 0; i < a->second.size(); ++i) acc += (double)a->second[i] * b->second[i];
  }
  return acc;
}
// y += alpha * x  (alpha = 1: AddTo, alpha = -1: Minus)
int tsb_ps_axpy(void* h, int64_t kx, int64_t ky, float alpha) {
  PS* p = static_cast<PS*>(h);
  if (key_len(p, kx) < 0 || key_len(p, kx) != key_len(p, ky)) return 1;
  for (auto& sh : p->shards) {
    std::lock_guard<std::mutex> g(sh.mu);
    auto& x = sh.store[kx];
    auto& y = sh.store[ky];
    for (size_t i = 0; i < x.size(); ++i) y[i] += alpha * x[i];
  }
  return 0;
}

// Heartbeats and dead-node detection.
int tsb_ps_heartbeat(void* h, int node) {
  PS* p = static_cast<PS*>(h);
  std::lock_guard<std::mutex> g(p->hb_mu);
  p->last_seen[node] = Clock::now();
  return 0;
}
int tsb_ps_dead_nodes(void* h, int timeout_ms, int* out, int max_out) {
  PS* p = static_cast<PS*>(h);
  std::lock_guard<std::mutex> g(p->hb_mu);
  const auto now = Clock::now();
  int n = 0;
  for (auto& kv : p->last_seen)
    if (std::chrono::duration_cast<std::chrono::milliseconds>(now - kv.second).count() > timeout_ms && n < max_out)
      out[n++] = kv.first;
  return n;
}

// out[0..3] = messages sent, dropped, re-sent, duplicates discarded
void tsb_ps_stats(void* h, int64_t* out) {
  PS* p = static_cast<PS*>(h);
  out[0] = p->sent; out[1] = p->dropped; out[2] = p->resent; out[3] = p->duplicates;
}

}  // extern "C"
