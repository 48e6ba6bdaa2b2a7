// TSplit planner: exact replay of a training step's memory behaviour under an HBM
// budget, and a greedy search over per-(micro-)tensor decisions.
//
// The reference ships only the hooks of its planner (per-op Profiler{time, input,
// output, workspace} structs, src/common/profiler.h:13-22, swap-cost constants,
// python/athena/profiler.py:8-14, micro-tensor views and the reuse allocation,
// src/common/c_runtime_api.cc:164-271); the planner modules themselves
// (microopPlanner / microopOptimizer) are absent.  This is a fresh design.
//
// Input: the schedule of a step, one entry per node in execution order.  When the
// executor has lowered the graph to micro-ops, every entry is a micro-op and every
// tensor a micro-tensor, so all decisions below are per micro-tensor.
//
// Decision per tensor: KEEP, SWAP (copy to pinned host memory, copy back before
// it is needed) or DROP (free, rebuild from its inputs when needed).  A tensor that
// is not KEEP leaves the device in EVERY idle gap between two consecutive uses that
// is long enough, not only between forward and backward: a swapped tensor is copied
// out once and fetched once per gap, a dropped one is rebuilt once per gap.
// Rebuilding a tensor uses its inputs, so each rebuild is a (virtual) use of them.
//
// derive():   decisions -> a list of events at schedule positions: evict (release
//             now / start the copy-out), free (the block of a copied-out tensor, at
//             the position where the copy is expected to be done; the compute stream
//             waits for the copy's event there, so the order of pool operations does
//             not depend on copy timing), prefetch (start the copy-in), plus the
//             final release position of every tensor.
// simulate(): replays the events against a REAL instance of the pool allocator
//             (same best-fit, two-ended placement as the executor's arena), with
//             three clocks (compute, H2D, D2H).  Because the executor performs the
//             same pool operations in the same order, "fits" is exact, fragmentation
//             included, and the predicted peak equals the measured one.
// search():   while the replay fails at some position, pick among the tensors that
//             are resident but idle there the one with the most bytes freed per
//             millisecond of added step time (swap while the host link has spare
//             time, otherwise rebuild), apply, replay again.  Afterwards hand
//             tensors back while the plan still fits and turn expensive rebuilds
//             into swaps where the link has room.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <cstdio>
#include <cstdlib>
#include <limits>
#include <utility>
#include <vector>


namespace {

enum { KEEP = 0, SWAP = 1, DROP = 2 };
enum { F_EVICTABLE = 1, F_RECOMPUTABLE = 2, F_PINNED = 4, F_EXTERNAL = 8 };
enum { EV_RELEASE = 0, EV_SWAPOUT = 1, EV_FREE = 2, EV_PREFETCH = 3 };


struct Graph {
  int n;
  const int64_t* out_bytes;
  const double* time_ms;
  const int* flags;
  const int* in_ptr;
  const int* in_idx;
  int64_t capacity;        // bytes of the simulated pool (the planning budget)
  double bw;               // host link, bytes per ms, per direction
  int min_gap = 3;         // positions between two uses before a tensor may leave in between
  std::vector<double> t0;  // prefix sums of time_ms: t0[i] = start of position i on an idle machine
  std::vector<std::vector<int>> real_uses;
  bool external(int t) const { return (flags[t] & F_EXTERNAL) != 0 || out_bytes[t] <= 0; }
  double xfer(int t) const { return (double)out_bytes[t] / bw; }
};

struct Event { int kind, pos, t; };

struct Fetch { int t, q, nu, free_pos; };

struct Events {
  std::vector<int> last_use;
  std::vector<std::vector<int>> uses;                  // per tensor, sorted, virtual uses included
  std::vector<std::vector<std::pair<int, int>>> gaps;  // per tensor: (evict after q, return at nu)
  std::vector<std::vector<Event>> after, before;       // per position
  std::vector<Fetch> fetches;                          // every return of a swapped tensor
  std::vector<Event> flat;
};

struct Result {
  double time_ms = 0, stall_ms = 0, rebuild_ms = 0;
  int64_t peak = 0, fail_need = 0, swap_out = 0, swap_in = 0, fail_free = 0, fail_largest = 0;
  int fail_pos = -1, rebuilds = 0, on_demand = 0, fail_allocs = 0;
  std::vector<int64_t> mem_at;
  std::vector<char> resident_at_fail;
  // one entry per planned allocation, in the order the executor performs them
  struct Block { int t; int born, died; int64_t size; int64_t offset; };
  std::vector<Block> blocks;
  std::vector<Event> prefetched;        // the prefetches that were really started, at their positions
  std::vector<int> rebuild_count;       // per tensor
  int64_t footprint = 0;
};

void prepare(Graph& g) {
  g.t0.assign(g.n + 1, 0.0);
  for (int i = 0; i < g.n; ++i) g.t0[i + 1] = g.t0[i] + g.time_ms[i];
  g.real_uses.assign(g.n, {});
  for (int i = 0; i < g.n; ++i)
    for (int e = g.in_ptr[i]; e < g.in_ptr[i + 1]; ++e) {
      auto& u = g.real_uses[g.in_idx[e]];
      if (u.empty() || u.back() != i) u.push_back(i);
    }
}

bool gap_ok(const Graph& g, int t, int cls, int q, int nu) {
  if (nu - q < g.min_gap) return false;
  if (cls == SWAP) return g.t0[nu] - g.t0[q + 1] >= 1.5 * g.xfer(t);   // the gap has to hide a round trip's half
  return true;
}

// `from[t]`: a tensor that is not KEEP leaves the device only in gaps that start at or after this position
// (its earlier, usually short, gaps stay resident).
void derive(const Graph& g, const std::vector<int>& cls, const std::vector<int>& from, Events& ev) {
  const int n = g.n;
  ev.last_use.assign(n, 0);
  ev.uses.assign(n, {});
  ev.gaps.assign(n, {});
  ev.after.assign(n, {});
  ev.before.assign(n, {});
  ev.fetches.clear();
  ev.flat.clear();
  std::vector<std::vector<int>> virt(n);
  for (int t = n - 1; t >= 0; --t) {
    std::vector<int>& u = ev.uses[t];
    u = g.real_uses[t];
    if (!virt[t].empty()) {
      u.insert(u.end(), virt[t].begin(), virt[t].end());
      std::sort(u.begin(), u.end());
      u.erase(std::unique(u.begin(), u.end()), u.end());
    }
    ev.last_use[t] = (g.flags[t] & F_PINNED) ? n : (u.empty() ? t : u.back());
    if (cls[t] == KEEP || g.external(t) || !(g.flags[t] & F_EVICTABLE)) continue;
    int q = t;
    for (int nu : u) {
      if (q >= from[t] && gap_ok(g, t, cls[t], q, nu)) ev.gaps[t].push_back({q, nu});
      q = nu;
    }
    if (cls[t] == DROP)
      for (auto& gp : ev.gaps[t])
        for (int e = g.in_ptr[t]; e < g.in_ptr[t + 1]; ++e) {
          const int in = g.in_idx[e];
          if (!g.external(in)) virt[in].push_back(gp.second);
        }
  }
  // evictions and planned frees of copied-out blocks
  struct Out { int t, q, nu; };
  std::vector<Out> outs;
  for (int t = 0; t < n; ++t) {
    bool first = true;
    for (auto& gp : ev.gaps[t]) {
      if (cls[t] == SWAP) {
        if (first) outs.push_back({t, gp.first, gp.second});
        else ev.after[gp.first].push_back({EV_RELEASE, gp.first, t});
        ev.fetches.push_back({t, gp.first, gp.second, first ? -1 : gp.first});
        first = false;
      } else {
        ev.after[gp.first].push_back({EV_RELEASE, gp.first, t});
      }
    }
  }
  std::sort(outs.begin(), outs.end(), [](const Out& a, const Out& b) { return a.q < b.q; });
  double td2h = 0;
  std::vector<int> free_pos(n, -1);
  for (auto& o : outs) {
    ev.after[o.q].push_back({EV_SWAPOUT, o.q, o.t});
    const double start = std::max(td2h, g.t0[o.q + 1]);
    const double done = start + g.xfer(o.t);
    td2h = done;
    int p = o.q;
    while (p + 1 < o.nu - 1 && g.t0[p + 1] < done) ++p;       // first position that ends after the copy
    free_pos[o.t] = p;
    ev.after[p].push_back({EV_FREE, p, o.t});
  }
  for (auto& f : ev.fetches)
    if (f.free_pos < 0) f.free_pos = free_pos[f.t];
  std::sort(ev.fetches.begin(), ev.fetches.end(), [](const Fetch& a, const Fetch& b) { return a.nu < b.nu; });
}

// Prefetch triggers: as early as the transfer needs to be hidden, but never so early that the tensor
// would sit in memory the schedule needs.  `mem` is the pool usage per position of a replay in which
// every swap-in happens on demand; each placed prefetch adds its bytes to the positions it spans.
void place_prefetch(const Graph& g, Events& ev, std::vector<int64_t> mem) {
  for (auto& b : ev.before) b.clear();
  double th2d = 0;
  int64_t largest = 0;
  for (int i = 0; i < g.n; ++i) largest = std::max(largest, g.external(i) ? 0 : g.out_bytes[i]);
  const int64_t limit = g.capacity - 2 * largest;      // early arrivals must not eat the room the next outputs need
  for (auto& f : ev.fetches) {
    const double need = g.xfer(f.t);
    const int64_t bytes = g.out_bytes[f.t];
    const int earliest = std::max(f.q, f.free_pos) + 1;
    int trig = f.nu;
    while (trig > earliest) {
      if (g.t0[f.nu] - std::max(th2d, g.t0[trig]) >= need * 1.2) break;
      if (mem[trig - 1] + bytes > limit) break;
      --trig;
    }
    th2d = std::max(th2d, g.t0[trig]) + need;
    for (int p = trig; p < f.nu; ++p) mem[p] += bytes;
    ev.before[trig].push_back({EV_PREFETCH, trig, f.t});
  }
}

void flatten(Events& ev) {
  ev.flat.clear();
  for (size_t p = 0; p < ev.after.size(); ++p) {
    for (auto& e : ev.before[p]) ev.flat.push_back(e);
    for (auto& e : ev.after[p]) ev.flat.push_back(e);
  }
}

struct Sim {
  const Graph& g;
  const std::vector<int>& cls;
  const Events& ev;
  const bool record;
  Result r;
  std::vector<int64_t> block;           // index into r.blocks (record mode) or 0, -1 = not resident
  std::vector<char> on_host, evicting, prefetched;
  std::vector<double> d2h_done, arrival;
  std::vector<int> queue, temps;
  std::vector<std::vector<int>> release_at;
  std::vector<int> leaving;             // leaving[t] == pos + 1: t is released after position pos
  std::vector<int> pinned_by_rebuild;   // inputs of rebuilds that are under way
  double tc = 0, th2d = 0, td2h = 0;
  int64_t in_use = 0;
  int ops = 0;                          // allocation / release counter: the time axis of the placement
  int n_alloc = 0;
  bool failed = false;
  const std::vector<std::pair<int, int>>* banned = nullptr;   // (tensor, trigger position) prefetches not to start
  std::vector<int> pf_pos;              // trigger position of the prefetch that brought a tensor in
  std::pair<int, int> cancel{-1, -1};   // at a failure: the unused prefetch whose use is farthest away

  Sim(const Graph& g_, const std::vector<int>& c, const Events& e, bool rec) : g(g_), cls(c), ev(e), record(rec) {
    block.assign(g.n, -1);
    on_host.assign(g.n, 0);
    evicting.assign(g.n, 0);
    prefetched.assign(g.n, 0);
    d2h_done.assign(g.n, 0.0);
    arrival.assign(g.n, 0.0);
    r.mem_at.assign(g.n, 0);
    r.rebuild_count.assign(g.n, 0);
    release_at.assign(g.n, {});
    leaving.assign(g.n, 0);
    pinned_by_rebuild.assign(g.n, 0);
    pf_pos.assign(g.n, -1);
    for (int t = 0; t < g.n; ++t)
      if (!g.external(t) && e.last_use[t] < g.n) release_at[e.last_use[t]].push_back(t);
  }

  int64_t used() const { return in_use; }
  static int64_t rounded(int64_t b) { return (b + 255) / 256 * 256; }

  bool alloc(int t, int pos) {
    const int64_t b = rounded(g.out_bytes[t]);
    if (in_use + b > g.capacity) {
      if (!failed) {
        failed = true;
        r.fail_pos = pos;
        r.fail_need = b;
        r.fail_free = g.capacity - in_use;
        r.fail_allocs = n_alloc;
        r.fail_largest = r.fail_free;
        r.resident_at_fail.assign(g.n, 0);
        for (int i = 0; i < g.n; ++i) r.resident_at_fail[i] = block[i] >= 0 && !evicting[i];
        int far = -1;
        for (int i = 0; i < g.n; ++i) {
          if (block[i] < 0 || !prefetched[i] || pf_pos[i] < 0) continue;
          int nu = g.n;
          for (int u : ev.uses[i]) if (u >= pos) { nu = u; break; }
          if (nu > pos && nu > far) { far = nu; cancel = {i, pf_pos[i]}; }
        }
      }
      return false;
    }
    in_use += b;
    ++ops;
    ++n_alloc;
    block[t] = 0;
    if (record && !(g.flags[t] & F_PINNED)) {
      block[t] = (int64_t)r.blocks.size();
      r.blocks.push_back({t, ops, std::numeric_limits<int>::max(), b, 0});
    }
    return true;
  }
  void release(int t) {
    if (block[t] < 0) return;
    if (on_host[t] && d2h_done[t] > tc) { r.stall_ms += d2h_done[t] - tc; tc = d2h_done[t]; }
    in_use -= rounded(g.out_bytes[t]);
    ++ops;
    if (record && !(g.flags[t] & F_PINNED)) r.blocks[block[t]].died = ops;
    block[t] = -1;
    evicting[t] = 0;
    prefetched[t] = 0;
  }
  bool swap_in(int t, int pos, bool prefetch) {
    if (!alloc(t, pos)) return false;
    const double start = std::max(std::max(th2d, tc), d2h_done[t]);
    th2d = start + g.xfer(t);
    arrival[t] = th2d;
    prefetched[t] = 1;
    r.swap_in += g.out_bytes[t];
    if (!prefetch) ++r.on_demand;
    return true;
  }
  bool ensure(int t, int pos) {
    if (g.external(t)) return true;
    if (block[t] >= 0) {
      evicting[t] = 0;          // needed again before its planned free: the block simply stays
      return true;
    }
    if (cls[t] == SWAP && on_host[t]) return swap_in(t, pos, false);
    for (int e = g.in_ptr[t]; e < g.in_ptr[t + 1]; ++e) {
      if (!ensure(g.in_idx[e], pos)) return false;
      ++pinned_by_rebuild[g.in_idx[e]];              // a nested rebuild must not send it away again
    }
    for (int e = g.in_ptr[t]; e < g.in_ptr[t + 1]; ++e) --pinned_by_rebuild[g.in_idx[e]];
    if (!alloc(t, pos)) return false;
    wait_inputs(t);
    tc += g.time_ms[t];
    r.rebuild_ms += g.time_ms[t];
    ++r.rebuilds;
    ++r.rebuild_count[t];
    temps.push_back(t);
    // inputs that were only needed for this rebuild (they leave after this position anyway and the node
    // itself does not read them) go at once, so a rebuild chain holds two links at a time, not all of them
    for (int e = g.in_ptr[t]; e < g.in_ptr[t + 1]; ++e) {
      const int u = g.in_idx[e];
      if (g.external(u) || block[u] < 0 || leaving[u] != pos + 1 || pinned_by_rebuild[u] > 0) continue;
      bool direct = false;
      for (int k = g.in_ptr[pos]; k < g.in_ptr[pos + 1]; ++k) direct |= (g.in_idx[k] == u);
      if (!direct) release(u);
    }
    return true;
  }
  void wait_inputs(int i) {
    for (int e = g.in_ptr[i]; e < g.in_ptr[i + 1]; ++e) {
      const int u = g.in_idx[e];
      if (prefetched[u]) {
        if (arrival[u] > tc) { r.stall_ms += arrival[u] - tc; tc = arrival[u]; }
        prefetched[u] = 0;
      }
    }
  }
  bool admit(int t, int pos) {
    int64_t largest = 0;
    int nu = pos;
    for (int u : ev.uses[t]) if (u >= pos) { nu = u; break; }
    for (int j = pos; j <= nu && j < g.n; ++j) largest = std::max(largest, g.external(j) ? 0 : g.out_bytes[j]);
    return in_use + rounded(g.out_bytes[t]) + 2 * largest <= g.capacity;
  }

  void run() {
    const int n = g.n;
    for (int pos = 0; pos < n && !failed; ++pos) {
      if (g.flags[pos] & F_EXTERNAL) { r.mem_at[pos] = used(); continue; }
      for (auto& e : ev.before[pos]) queue.push_back(e.t);
      if (!queue.empty()) {
        std::vector<int> waiting;
        for (int t : queue) {
          if (!on_host[t] || block[t] >= 0) continue;
          if (banned && std::find(banned->begin(), banned->end(), std::make_pair(t, pos)) != banned->end()) continue;
          if (!waiting.empty() || !admit(t, pos)) { waiting.push_back(t); continue; }
          swap_in(t, pos, true);
          pf_pos[t] = pos;
          if (record) r.prefetched.push_back({EV_PREFETCH, pos, t});
        }
        queue.swap(waiting);
      }
      temps.clear();
      for (auto& e : ev.after[pos]) if (e.kind == EV_RELEASE) leaving[e.t] = pos + 1;
      for (int t : release_at[pos]) leaving[t] = pos + 1;
      bool ok = true;
      for (int e = g.in_ptr[pos]; e < g.in_ptr[pos + 1] && ok; ++e) ok = ensure(g.in_idx[e], pos);
      if (!ok) break;
      if (g.out_bytes[pos] > 0 && !alloc(pos, pos)) break;
      wait_inputs(pos);
      tc += g.time_ms[pos];
      const int64_t u = used();
      r.mem_at[pos] = u;
      if (u > r.peak) r.peak = u;
      for (auto& e : ev.after[pos]) {
        const int t = e.t;
        if (block[t] < 0) continue;
        if (e.kind == EV_SWAPOUT) {
          if (!on_host[t]) {
            const double start = std::max(td2h, tc);
            td2h = start + g.xfer(t);
            d2h_done[t] = td2h;
            on_host[t] = 1;
            r.swap_out += g.out_bytes[t];
          }
          evicting[t] = 1;
        } else if (e.kind == EV_FREE) {
          if (evicting[t]) release(t);
        } else if (e.kind == EV_RELEASE) {
          release(t);
        }
      }
      for (int t : release_at[pos]) {      // last (real or virtual) use was here
        release(t);
        on_host[t] = 0;
      }
    }
    r.time_ms = std::max(tc, std::max(th2d, td2h));
  }
};

// A prefetch that arrives early holds memory the schedule may need before the tensor is used.  When the
// replay fails while such a tensor sits unused, that prefetch is struck (the tensor then comes on demand,
// or by a later trigger) and the replay starts over, so early arrivals never are what makes a plan fail.
Result simulate(const Graph& g, const std::vector<int>& cls, const Events& ev, bool record = false) {
  std::vector<std::pair<int, int>> banned;
  for (int round = 0;; ++round) {
    Sim s(g, cls, ev, record);
    s.banned = &banned;
    s.run();
    if (s.r.fail_pos < 0 || s.cancel.first < 0 || round >= 64) return std::move(s.r);
    banned.push_back(s.cancel);
  }
}

// Offline placement of the recorded allocations (each lives from its allocation to its release on the
// executor's operation counter): largest first, each at the lowest offset that is free of the blocks
// already placed whose lifetimes overlap its own.  Because the executor replays exactly this sequence,
// every block can be given its address ahead of time: no allocator runs during a step and there is no
// fragmentation beyond what this packing leaves.  Returns the footprint (highest end offset).
int64_t place_in_order(std::vector<Result::Block>& blocks, const std::vector<int>& order) {
  const int n = (int)blocks.size();
  std::vector<int> placed;
  placed.reserve(n);
  int64_t footprint = 0;
  std::vector<std::pair<int64_t, int64_t>> busy;
  for (int i : order) {
    Result::Block& b = blocks[i];
    busy.clear();
    for (int j : placed) {
      const Result::Block& o = blocks[j];
      if (o.born < b.died && b.born < o.died) busy.push_back({o.offset, o.offset + o.size});
    }
    std::sort(busy.begin(), busy.end());
    int64_t off = 0;
    for (auto& iv : busy) {
      if (iv.first - off >= b.size) break;
      off = std::max(off, iv.second);
    }
    b.offset = off;
    footprint = std::max(footprint, off + b.size);
    placed.push_back(i);
  }
  return footprint;
}

// Three placement orders are tried (largest block first; largest size x lifetime first; longest lifetime
// first) and the tightest packing is kept.
int64_t place(std::vector<Result::Block>& blocks) {
  const int n = (int)blocks.size();
  std::vector<int> order(n);
  auto life = [&](int i) { return (int64_t)blocks[i].died - blocks[i].born; };
  int64_t best = std::numeric_limits<int64_t>::max();
  std::vector<int64_t> best_off(n, 0);
  for (int variant = 0; variant < 3; ++variant) {
    for (int i = 0; i < n; ++i) order[i] = i;
    std::sort(order.begin(), order.end(), [&](int a, int b) {
      if (variant == 0) {
        if (blocks[a].size != blocks[b].size) return blocks[a].size > blocks[b].size;
        return life(a) > life(b);
      }
      if (variant == 1) {
        const double aa = (double)blocks[a].size * (double)life(a), bb = (double)blocks[b].size * (double)life(b);
        if (aa != bb) return aa > bb;
        return a < b;
      }
      if (life(a) != life(b)) return life(a) > life(b);
      return blocks[a].size > blocks[b].size;
    });
    const int64_t fp = place_in_order(blocks, order);
    if (fp < best) {
      best = fp;
      for (int i = 0; i < n; ++i) best_off[i] = blocks[i].offset;
    }
  }
  for (int i = 0; i < n; ++i) blocks[i].offset = best_off[i];
  return best;
}

// decisions -> events -> replay.  Two replays: one with every swap-in on demand (its memory curve tells
// how early each prefetch may start), then the real one.
Result evaluate(const Graph& g, const std::vector<int>& cls, const std::vector<int>& from, Events& ev,
                bool record = false) {
  derive(g, cls, from, ev);
  if (!ev.fetches.empty()) {
    Result jit = simulate(g, cls, ev);
    place_prefetch(g, ev, jit.mem_at);
  }
  flatten(ev);
  Result r = simulate(g, cls, ev, record);
  if (record) {
    // the executor follows the plan literally: keep only the prefetches the replay really started, at the
    // positions where it started them, and give every allocation its address
    for (auto& b : ev.before) b.clear();
    for (auto& e : r.prefetched) ev.before[e.pos].push_back(e);
    flatten(ev);
    r.footprint = place(r.blocks);
  }
  return r;
}

double rebuild_cost(const Graph& g, const std::vector<int>& cls, int t, int depth = 0) {
  double ms = g.time_ms[t];
  if (depth > 48) return ms;
  for (int e = g.in_ptr[t]; e < g.in_ptr[t + 1]; ++e) {
    const int u = g.in_idx[e];
    if (g.external(u)) continue;
    if (cls[u] == DROP) ms += rebuild_cost(g, cls, u, depth + 1);
    else if (cls[u] == SWAP) ms += 0.5 * g.xfer(u);
  }
  return ms;
}

void write_out(const Graph& g, const std::vector<int>& cls, const Events& ev, const Result& r, int* cls_out,
               int* last_use_out, int ev_cap, int* ev_kind, int* ev_pos, int* ev_tensor, int* ev_count,
               int alloc_cap, int* alloc_tensor, int64_t* alloc_offset, int* alloc_count, double* summary,
               int64_t* mem_at, int* rebuild_count = nullptr) {
  if (cls_out) std::memcpy(cls_out, cls.data(), sizeof(int) * g.n);
  if (last_use_out) std::memcpy(last_use_out, ev.last_use.data(), sizeof(int) * g.n);
  int c = 0;
  for (auto& e : ev.flat) {
    if (c >= ev_cap) break;
    ev_kind[c] = e.kind; ev_pos[c] = e.pos; ev_tensor[c] = e.t;
    ++c;
  }
  if (ev_count) *ev_count = (int)ev.flat.size();
  c = 0;
  for (auto& b : r.blocks) {
    if (c >= alloc_cap) break;
    alloc_tensor[c] = b.t; alloc_offset[c] = b.offset;
    ++c;
  }
  if (alloc_count) *alloc_count = (int)r.blocks.size();
  summary[0] = r.time_ms; summary[1] = (double)r.peak; summary[2] = r.fail_pos; summary[3] = r.stall_ms;
  summary[4] = (double)r.fail_need; summary[5] = (double)r.swap_out; summary[6] = (double)r.swap_in;
  summary[7] = r.rebuild_ms; summary[8] = r.rebuilds; summary[9] = r.on_demand;
  summary[10] = (double)r.fail_free; summary[11] = (double)r.footprint;
  if (mem_at) std::memcpy(mem_at, r.mem_at.data(), sizeof(int64_t) * g.n);
  if (rebuild_count) std::memcpy(rebuild_count, r.rebuild_count.data(), sizeof(int) * g.n);
}

int64_t pinned_bytes(const Graph& g) {
  int64_t b = 0;
  for (int i = 0; i < g.n; ++i)
    if ((g.flags[i] & F_PINNED) && !g.external(i)) b += (g.out_bytes[i] + 255) / 256 * 256;
  return b;
}

}  // namespace

extern "C" {

// Replay the plan (cls = KEEP/SWAP/DROP per schedule entry, from = first position from which a non-KEEP
// tensor's gaps are evicted; may be null = from the start) in `capacity` bytes.
// flags: 1 = may be evicted, 2 = may be rebuilt, 4 = never released (a result; allocated by the caller outside
// the placed region, but counted against the capacity), 8 = external (feeds, parameters).
// Outputs: last_use[n]; the event list (kind 0 release / 1 start copy-out / 2 free copied-out block / 3 prefetch,
// position, tensor) in execution order, events "before" a position first; the allocation list in execution
// order (tensor, byte offset inside the placed region); summary[12] = step ms, peak bytes in use, first failing
// position (-1 = fits), stall ms, bytes of the failed request, bytes copied out, bytes copied in, rebuild ms,
// rebuilt tensors, on-demand swap-ins, free bytes at the failure, footprint of the placed region; mem_at[n]
// (may be null) = bytes in use at every position; rebuild_count[n] (may be null) = times each tensor is rebuilt.
// Returns 0, or 6 when an output array is too small (the counts then hold the required sizes).
int tsb_plan2_simulate(int n, const int64_t* out_bytes, const double* time_ms, const int* flags, const int* in_ptr,
                       const int* in_idx, int64_t capacity, int64_t min_gap, double bw_bytes_per_ms,
                       const int* cls_in, const int* from_in, int* last_use_out, int ev_cap, int* ev_kind,
                       int* ev_pos, int* ev_tensor, int* ev_count, int alloc_cap, int* alloc_tensor,
                       int64_t* alloc_offset, int* alloc_count, double* summary, int64_t* mem_at,
                       int* rebuild_count) {
  if (n <= 0 || !summary) return 1;
  Graph g{n, out_bytes, time_ms, flags, in_ptr, in_idx, capacity, bw_bytes_per_ms};
  g.min_gap = min_gap > 0 ? (int)min_gap : 3;
  prepare(g);
  std::vector<int> cls(cls_in, cls_in + n), from(n, 0);
  if (from_in) from.assign(from_in, from_in + n);
  Events ev;
  Result r = evaluate(g, cls, from, ev, true);
  write_out(g, cls, ev, r, nullptr, last_use_out, ev_cap, ev_kind, ev_pos, ev_tensor, ev_count, alloc_cap,
            alloc_tensor, alloc_offset, alloc_count, summary, mem_at, rebuild_count);
  return ((int)ev.flat.size() > ev_cap || (int)r.blocks.size() > alloc_cap) ? 6 : 0;
}

// Search a plan.  Same outputs as tsb_plan2_simulate plus cls_out[n] and from_out[n].  Returns 0 when the plan
// fits, 5 when no plan was found (the outputs then describe the best attempt), 6 when the event arrays are too
// small.
int tsb_plan2_search(int n, const int64_t* out_bytes, const double* time_ms, const int* flags, const int* in_ptr,
                     const int* in_idx, int64_t capacity, int64_t min_gap, double bw_bytes_per_ms,
                     int allow_swap, int* cls_out, int* from_out, int* last_use_out, int ev_cap, int* ev_kind,
                     int* ev_pos, int* ev_tensor, int* ev_count, int alloc_cap, int* alloc_tensor,
                     int64_t* alloc_offset, int* alloc_count, double* summary, int64_t* mem_at,
                     int* rebuild_count) {
  if (n <= 0 || !summary) return 1;
  Graph g{n, out_bytes, time_ms, flags, in_ptr, in_idx, capacity, bw_bytes_per_ms};
  g.min_gap = min_gap > 0 ? (int)min_gap : 3;
  prepare(g);
  const int NEVER = std::numeric_limits<int>::max();
  std::vector<int> cls(n, KEEP), from(n, NEVER);
  Events ev;
  Result r;
  // The search counts bytes; the placement of the final plan may need a little more than its peak.  When
  // the footprint overshoots the real capacity, search again with the capacity reduced by the overshoot.
  for (int round = 0; round < 4; ++round) {
  r = evaluate(g, cls, from, ev);
  const double total_ms = g.t0[n];
  double link_ms = 0.0;                       // copy time (one direction) already committed to swaps
  std::vector<char> no_drop(n, 0), no_swap(n, 0);
  const bool debug = getenv("TSB_PLAN_DEBUG") != nullptr;
  // refinement trials after a plan fits (each is a full replay); TSB_PLAN_REFINE overrides
  const int refine_tries = getenv("TSB_PLAN_REFINE") ? atoi(getenv("TSB_PLAN_REFINE")) : 600;
  int guard = 0;
  bool retried = false;
  while (r.fail_pos >= 0 && guard++ < 16 * n) {
    const int pos = r.fail_pos;
    struct Cand { double score; int t; int cls; int q; };
    std::vector<Cand> cands;
    for (int t = 0; t < n; ++t) {
      if (!(g.flags[t] & F_EVICTABLE) || g.external(t) || !r.resident_at_fail[t]) continue;
      // the gap of t that spans `pos`
      int q = t, nu = -1;
      for (int u : ev.uses[t]) {
        if (u >= pos) { nu = u; break; }
        q = u;
      }
      if (nu < 0 || nu == pos || q >= pos) continue;
      if (cls[t] != KEEP && from[t] <= q) continue;          // this gap is evicted already (too short to count)
      bool is_input = false;
      for (int e = g.in_ptr[pos]; e < g.in_ptr[pos + 1]; ++e) is_input |= (g.in_idx[e] == t);
      if (is_input) continue;
      int returns = 0, qq = t;
      for (int u : ev.uses[t]) { if (qq >= q && u - qq >= g.min_gap) ++returns; qq = u; }
      returns = std::max(1, returns);
      const bool may_swap = cls[t] == KEEP || cls[t] == SWAP, may_drop = cls[t] == KEEP || cls[t] == DROP;
      // a copy-out only helps here when it can finish between the eviction and the failing position
      if (allow_swap && may_swap && !no_swap[t] && gap_ok(g, t, SWAP, q, nu) &&
          (cls[t] == SWAP || g.t0[pos] - g.t0[q + 1] >= g.xfer(t))) {
        const double x = g.xfer(t);
        const bool room = link_ms + x * returns <= 0.8 * total_ms;
        const double cost = room ? 0.03 * x * returns : x * (1 + returns);
        cands.push_back({(double)g.out_bytes[t] / (cost + 1e-3), t, SWAP, q});
      }
      if ((g.flags[t] & F_RECOMPUTABLE) && may_drop && !no_drop[t] && gap_ok(g, t, DROP, q, nu)) {
        const double cost = rebuild_cost(g, cls, t) * returns;
        cands.push_back({(double)g.out_bytes[t] / (cost + 1e-3), t, DROP, q});
      }
    }
    std::sort(cands.begin(), cands.end(), [](const Cand& a, const Cand& b) { return a.score > b.score; });
    bool accepted = false;
    auto progress = [&](const Result& trial) {
      // further along: a later position, or at the same one more of its allocations done / more bytes free
      return trial.fail_pos < 0 || trial.fail_pos > pos ||
             (trial.fail_pos == pos && (trial.fail_allocs > r.fail_allocs ||
                                        (trial.fail_allocs == r.fail_allocs && trial.fail_free > r.fail_free)));
    };
    for (size_t ci = 0; ci < cands.size() && ci < 256 && !accepted; ++ci) {
      const int t = cands[ci].t;
      std::vector<std::pair<int, std::pair<int, int>>> undo{{t, {cls[t], from[t]}}};
      cls[t] = cands[ci].cls;
      from[t] = std::min(from[t], cands[ci].q);
      Events tev;
      Result trial = evaluate(g, cls, from, tev);
      bool better = progress(trial);
      if (!better && cands[ci].cls == DROP) {
        // Dropping t alone only moves the bytes to the inputs its rebuild keeps alive.  Drop the chain:
        // every input (recursively) that stays resident only for that rebuild, down to tensors that are
        // small next to t, external or not rebuildable.
        std::vector<int> frontier{t};
        for (int depth = 0; depth < 8 && !frontier.empty(); ++depth) {
          std::vector<int> next;
          for (int x : frontier)
            for (int e = g.in_ptr[x]; e < g.in_ptr[x + 1]; ++e) {
              const int u = g.in_idx[e];
              if (g.external(u) || cls[u] == SWAP) continue;
              if (!(g.flags[u] & F_EVICTABLE) || !(g.flags[u] & F_RECOMPUTABLE)) continue;
              if (g.out_bytes[u] * 3 <= g.out_bytes[t]) continue;
              int last_before = u;                               // last real use before the failing position
              bool used_at_or_after = false;
              for (int w : g.real_uses[u]) {
                if (w < pos) last_before = w; else used_at_or_after = true;
              }
              if (cls[u] == DROP && from[u] <= last_before) continue;      // already evicted over this stretch
              (void)used_at_or_after;
              undo.push_back({u, {cls[u], from[u]}});
              cls[u] = DROP;
              from[u] = std::min(from[u], last_before);
              next.push_back(u);
            }
          frontier.swap(next);
        }
        if (undo.size() > 1) {
          trial = evaluate(g, cls, from, tev);
          better = progress(trial);
        }
      }
      if (debug)
        fprintf(stderr, "pos %d cand t=%d cls=%d q=%d chain %zu score %.3g -> fail %d free %lld (was %lld) %s\n", pos, t,
                cands[ci].cls, cands[ci].q, undo.size(), cands[ci].score, trial.fail_pos, (long long)trial.fail_free,
                (long long)r.fail_free, better ? "ACCEPT" : "reject");
      if (better) {
        if (cands[ci].cls == SWAP) link_ms += g.xfer(t) * std::max<size_t>(1, tev.gaps[t].size());
        r = std::move(trial);
        ev = std::move(tev);
        accepted = true;
      } else {
        (cands[ci].cls == DROP ? no_drop : no_swap)[t] = 1;
        for (auto& u : undo) { cls[u.first] = u.second.first; from[u.first] = u.second.second; }
      }
    }
    if (!accepted && !retried) {        // decisions taken since may have made a rejected candidate useful
      retried = true;
      std::fill(no_drop.begin(), no_drop.end(), 0);
      std::fill(no_swap.begin(), no_swap.end(), 0);
      continue;
    }
    if (accepted) retried = false;
    if (!accepted) break;       // what is resident at the failing position is all in use there
  }
  if (r.fail_pos < 0) {
    // 1. hand tensors back while the plan still fits and does not get slower, most expensive first
    std::vector<std::pair<double, int>> evicted;
    for (int t = 0; t < n; ++t) {
      if (cls[t] == KEEP) continue;
      const double cost = cls[t] == DROP ? rebuild_cost(g, cls, t) * std::max<size_t>(1, ev.gaps[t].size())
                                         : g.xfer(t) * (1 + ev.gaps[t].size()) * 0.25;
      evicted.push_back({cost, t});
    }
    std::sort(evicted.begin(), evicted.end(),
              [](const std::pair<double, int>& a, const std::pair<double, int>& b) { return a.first > b.first; });
    int tries = 0;
    for (auto& e : evicted) {
      if (++tries > refine_tries) break;
      const int t = e.second, was = cls[t], was_from = from[t];
      cls[t] = KEEP;
      from[t] = NEVER;
      Events tev;
      Result trial = evaluate(g, cls, from, tev);
      if (trial.fail_pos < 0 && trial.time_ms <= r.time_ms + 1e-9) { r = std::move(trial); ev = std::move(tev); }
      else { cls[t] = was; from[t] = was_from; }
    }
    // 2. expensive rebuilds become swaps where that shortens the step
    if (allow_swap) {
      std::vector<std::pair<double, int>> dropped;
      for (int t = 0; t < n; ++t)
        if (cls[t] == DROP) dropped.push_back({rebuild_cost(g, cls, t) * std::max<size_t>(1, ev.gaps[t].size()), t});
      std::sort(dropped.begin(), dropped.end(),
                [](const std::pair<double, int>& a, const std::pair<double, int>& b) { return a.first > b.first; });
      tries = 0;
      for (auto& e : dropped) {
        if (++tries > refine_tries / 2) break;
        const int t = e.second;
        cls[t] = SWAP;
        Events tev;
        Result trial = evaluate(g, cls, from, tev);
        if (!tev.gaps[t].empty() && trial.fail_pos < 0 && trial.time_ms < r.time_ms - 1e-6) {
          r = std::move(trial);
          ev = std::move(tev);
        } else {
          cls[t] = DROP;
        }
      }
    }
  }
  r = evaluate(g, cls, from, ev, true);
  if (r.fail_pos >= 0) break;
  const int64_t room = capacity - pinned_bytes(g);
  if (r.footprint <= room) break;
  if (round == 3) { r.fail_pos = 0; break; }                 // could not be packed: reported as not fitting
  g.capacity = (int64_t)((double)g.capacity * (double)room / (double)r.footprint * 0.995);
  }
  for (int t = 0; t < n; ++t)
    if (from[t] == NEVER) from[t] = 0;
  if (from_out) std::memcpy(from_out, from.data(), sizeof(int) * n);
  write_out(g, cls, ev, r, cls_out, last_use_out, ev_cap, ev_kind, ev_pos, ev_tensor, ev_count, alloc_cap,
            alloc_tensor, alloc_offset, alloc_count, summary, mem_at, rebuild_count);
  if ((int)ev.flat.size() > ev_cap || (int)r.blocks.size() > alloc_cap) return 6;
  return r.fail_pos < 0 ? 0 : 5;
}

}  // extern "C"
