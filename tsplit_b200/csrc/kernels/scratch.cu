// Registry of the library-owned device scratch buffers (see scratch.h).
#include "scratch.h"

#include <map>
#include <mutex>
#include <tuple>
#include <vector>

namespace {

struct Buf {
  void* ptr = nullptr;
  size_t bytes = 0;
};
std::mutex g_mu;
std::map<std::tuple<int, cudaStream_t, int>, Buf> g_table;
std::vector<std::pair<int, Buf>> g_parked;        // (device, replaced buffer)
long long g_total = 0;

}  // namespace

namespace tsb_scratch {

void* get(cudaStream_t stream, int tag, size_t bytes, size_t floor_bytes) {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> g(g_mu);
  Buf& b = g_table[std::make_tuple(dev, stream, tag)];
  if (b.bytes >= bytes && b.ptr) return b.ptr;
  const size_t want = bytes < floor_bytes ? floor_bytes : bytes;
  void* fresh = nullptr;
  if (cudaMalloc(&fresh, want) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (b.ptr) g_parked.push_back({dev, b});         // work queued on the stream may still use it
  b.ptr = fresh;
  b.bytes = want;
  g_total += (long long)want;
  return b.ptr;
}

}  // namespace tsb_scratch

extern "C" {

long long tsb_scratch_bytes() {
  std::lock_guard<std::mutex> g(g_mu);
  return g_total;
}

long long tsb_scratch_trim() {
  std::lock_guard<std::mutex> g(g_mu);
  int cur = 0;
  cudaGetDevice(&cur);
  long long freed = 0;
  for (auto& p : g_parked) {
    cudaSetDevice(p.first);
    if (cudaFree(p.second.ptr) == cudaSuccess) freed += (long long)p.second.bytes;
  }
  g_parked.clear();
  cudaSetDevice(cur);
  g_total -= freed;
  return freed;
}

}  // extern "C"
