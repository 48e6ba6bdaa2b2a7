// Capped best-fit offset allocator with coalescing.
//
// The pool hands out byte offsets into one arena that the caller owns (a device
// allocation sized to the HBM budget, or host memory for the simulated device),
// so the same code serves the GPU executors and the CPU test-suite.  Semantics
// follow the reference's (unplugged) DLMemoryManager — one up-front reservation,
// best fit, split on allocation, merge with free neighbours on release, usage
// and try-allocate queries (src/cuda_common/gpu_memory_manager.cc:70-284) — with
// an ordered size index instead of power-of-two bins and typed error codes
// instead of exit().
#include <cstdint>
#include <map>
#include <mutex>
#include <set>
#include <utility>

namespace {

struct Pool {
  int64_t capacity;
  int64_t align;
  int64_t used = 0;
  int64_t peak = 0;
  int64_t n_alloc = 0;
  int64_t n_fail = 0;
  std::map<int64_t, std::pair<int64_t, bool>> blocks;   // offset -> (size, is_free)
  std::set<std::pair<int64_t, int64_t>> free_by_size;   // (size, offset)
  std::mutex mu;
};

int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

}  // namespace

extern "C" {

void* tsb_pool_create(int64_t capacity, int64_t alignment) {
  if (capacity <= 0) return nullptr;
  Pool* p = new Pool();
  p->align = alignment > 0 ? alignment : 256;
  p->capacity = capacity / p->align * p->align;
  p->blocks[0] = {p->capacity, true};
  p->free_by_size.insert({p->capacity, 0});
  return p;
}

void tsb_pool_destroy(void* h) { delete static_cast<Pool*>(h); }

// 0 = ok (offset written), 5 = does not fit
int tsb_pool_alloc(void* h, int64_t bytes, int64_t* offset) {
  Pool* p = static_cast<Pool*>(h);
  if (!p || bytes < 0 || !offset) return 1;
  const int64_t need = round_up(bytes > 0 ? bytes : 1, p->align);
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->free_by_size.lower_bound({need, -1});
  if (it == p->free_by_size.end()) {
    ++p->n_fail;
    return 5;
  }
  const int64_t size = it->first, off = it->second;
  p->free_by_size.erase(it);
  if (size > need) {
    p->blocks[off] = {need, false};
    p->blocks[off + need] = {size - need, true};
    p->free_by_size.insert({size - need, off + need});
  } else {
    p->blocks[off].second = false;
  }
  p->used += need;
  if (p->used > p->peak) p->peak = p->used;
  ++p->n_alloc;
  *offset = off;
  return 0;
}

// Same, but carves the block from the TOP of the highest free range that fits.
// Long-lived tensors (results, parameter gradients) go there so they do not
// fragment the low end where short-lived activations churn.
int tsb_pool_alloc_high(void* h, int64_t bytes, int64_t* offset) {
  Pool* p = static_cast<Pool*>(h);
  if (!p || bytes < 0 || !offset) return 1;
  const int64_t need = round_up(bytes > 0 ? bytes : 1, p->align);
  std::lock_guard<std::mutex> g(p->mu);
  for (auto it = p->blocks.rbegin(); it != p->blocks.rend(); ++it) {
    if (!it->second.second || it->second.first < need) continue;
    const int64_t off = it->first, size = it->second.first;
    p->free_by_size.erase({size, off});
    if (size > need) {
      p->blocks[off] = {size - need, true};
      p->free_by_size.insert({size - need, off});
      p->blocks[off + size - need] = {need, false};
      *offset = off + size - need;
    } else {
      p->blocks[off].second = false;
      *offset = off;
    }
    p->used += need;
    if (p->used > p->peak) p->peak = p->used;
    ++p->n_alloc;
    return 0;
  }
  ++p->n_fail;
  return 5;
}

int tsb_pool_free(void* h, int64_t offset) {
  Pool* p = static_cast<Pool*>(h);
  if (!p) return 1;
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->blocks.find(offset);
  if (it == p->blocks.end() || it->second.second) return 1;   // unknown block or double free
  int64_t off = it->first, size = it->second.first;
  p->used -= size;
  // merge with the next block
  auto nx = std::next(it);
  if (nx != p->blocks.end() && nx->second.second) {
    p->free_by_size.erase({nx->second.first, nx->first});
    size += nx->second.first;
    p->blocks.erase(nx);
  }
  // merge with the previous block
  if (it != p->blocks.begin()) {
    auto pv = std::prev(it);
    if (pv->second.second) {
      p->free_by_size.erase({pv->second.first, pv->first});
      off = pv->first;
      size += pv->second.first;
      p->blocks.erase(it);
      it = pv;
    }
  }
  it->second = {size, true};
  p->free_by_size.insert({size, off});
  return 0;
}

// Pack every used block towards offset 0 (order preserved) so that the free space becomes one
// range.  Writes up to `max_moves` relocations (old offset, new offset, size), lowest first, and
// returns their number; the caller moves the bytes in that order (each move goes downwards).
int tsb_pool_compact(void* h, int64_t* old_off, int64_t* new_off, int64_t* sizes, int max_moves) {
  Pool* p = static_cast<Pool*>(h);
  if (!p) return 0;
  std::lock_guard<std::mutex> g(p->mu);
  std::map<int64_t, std::pair<int64_t, bool>> packed;
  int64_t cursor = 0;
  int n = 0;
  for (auto& kv : p->blocks) {
    if (kv.second.second) continue;
    if (kv.first != cursor) {
      if (n >= max_moves) {          // table too small: keep the remaining blocks where they are
        cursor = kv.first;
      } else {
        old_off[n] = kv.first; new_off[n] = cursor; sizes[n] = kv.second.first;
        ++n;
      }
    }
    packed[cursor] = {kv.second.first, false};
    cursor += kv.second.first;
  }
  p->free_by_size.clear();
  // rebuild the free ranges between / after the packed blocks
  std::map<int64_t, std::pair<int64_t, bool>> rebuilt;
  int64_t pos = 0;
  for (auto& kv : packed) {
    if (kv.first > pos) { rebuilt[pos] = {kv.first - pos, true}; p->free_by_size.insert({kv.first - pos, pos}); }
    rebuilt[kv.first] = kv.second;
    pos = kv.first + kv.second.first;
  }
  if (pos < p->capacity) { rebuilt[pos] = {p->capacity - pos, true}; p->free_by_size.insert({p->capacity - pos, pos}); }
  p->blocks.swap(rebuilt);
  return n;
}

// 1 when a block of `bytes` could be allocated right now
int tsb_pool_try(void* h, int64_t bytes) {
  Pool* p = static_cast<Pool*>(h);
  if (!p) return 0;
  const int64_t need = round_up(bytes > 0 ? bytes : 1, p->align);
  std::lock_guard<std::mutex> g(p->mu);
  return p->free_by_size.lower_bound({need, -1}) != p->free_by_size.end() ? 1 : 0;
}

// out[0..6] = capacity, used, free_total, largest_free, peak_used, alloc_count, fail_count
void tsb_pool_stats(void* h, int64_t* out) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  out[0] = p->capacity;
  out[1] = p->used;
  out[2] = p->capacity - p->used;
  out[3] = p->free_by_size.empty() ? 0 : p->free_by_size.rbegin()->first;
  out[4] = p->peak;
  out[5] = p->n_alloc;
  out[6] = p->n_fail;
}

void tsb_pool_reset_peak(void* h) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  p->peak = p->used;
}

// size of the block at `offset` (0 when unknown)
int64_t tsb_pool_block_size(void* h, int64_t offset) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->blocks.find(offset);
  return it == p->blocks.end() ? 0 : it->second.first;
}

}  // extern "C"
