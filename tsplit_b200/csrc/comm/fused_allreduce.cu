// Fused gradient all-reduce + 1/N scale + optimizer update + parameter broadcast
// over NVLink peer memory, ONE kernel per bucket.
//
// Every rank holds its full gradient bucket and the full parameter bucket in
// peer-mapped (symmetric) memory.  Rank r owns elements [r*S/N, (r+1)*S/N):
//   phase 0  flag exchange: "my gradients are complete" (st.release.sys to every
//            peer's flag word, bounded ld.acquire.sys spin on my own words)
//   phase 1  for the owned shard: load the N peers' gradient values with plain
//            16-byte peer loads (or one multimem.ld_reduce through the NVSwitch
//            when a multicast mapping is given), sum in fixed rank order, scale
//            by 1/N, apply SGD / momentum / Nesterov / AdaGrad / Adam to the owned
//            parameter shard, and store the NEW PARAMETERS to all N peers
//            (or one multimem.st)
//   phase 2  flag exchange: "my shard is written everywhere"
// so gradients cross the links once (reduce-scatter) and parameters once
// (all-gather), and the optimizer state is sharded N ways.  No TMA, no multicast
// TMA: only ld/st/multimem on generic pointers.
//
// Every spin is bounded (about one second).  When the first exchange runs out, the
// kernel records a status word and the whole grid returns before the reduction: the
// parameters and the optimizer state of this rank stay as they were, and the host
// raises a timeout error.
//
// Role in the reference: ncclAllReduce per gradient tensor followed by a stream
// sync (src/communication/mpi_nccl_communication.cu:101-120) and a separate
// optimizer launch per parameter (src/ops/Optimizers.cu).
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cg = cooperative_groups;

#define TSB_OK 0
#define TSB_ERR_ARG 1
#define TSB_ERR_LAUNCH 3
#define TSB_ERR_TIMEOUT 4

namespace {

constexpr int MAX_RANKS = 16;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;

struct Args {
  const float* grad[MAX_RANKS];   // peer pointers to the gradient bucket
  float* param[MAX_RANKS];        // peer pointers to the parameter bucket
  uint32_t* flags[MAX_RANKS];     // peer pointers to the flag words: [2 * MAX_RANKS] per rank
  const float* grad_mc;           // multicast address of the gradient bucket (or null)
  float* param_mc;                // multicast address of the parameter bucket (or null)
  float* slot1;                   // local optimizer state for the owned shard (shard-local indexing)
  float* slot2;
  long long n;                    // bucket elements (multiple of 4)
  long long lo, hi;               // owned shard
  int rank, world, kind;
  uint32_t epoch;
  float h[8];
  int* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_peer(float* p, const float4& v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ float4 multimem_ld_reduce(const float* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(float* p, const float4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}

template <int KIND>
__device__ __forceinline__ void opt_one(float& p, float g, float& s1, float& s2, const float* h) {
  if (KIND == 0) {
    p -= h[0] * g;
  } else if (KIND == 1) {
    s1 = h[1] * s1 - h[0] * g;
    p += s1;
  } else if (KIND == 2) {
    const float lr_g = -h[0] * g;
    s1 = h[1] * (s1 + lr_g);
    p += s1 + lr_g;
  } else if (KIND == 3) {
    s1 += g * g;
    p -= h[0] * g / (sqrtf(s1) + h[1]);
  } else {
    s1 = h[1] * s1 + (1.f - h[1]) * g;
    s2 = h[2] * s2 + (1.f - h[2]) * g * g;
    p -= h[0] * (s1 / (1.f - h[3])) / (sqrtf(s2 / (1.f - h[4])) + h[5]);
  }
}

// Epoch of the last call on this device whose first exchange ran out of time.  Written by block 0
// before the grid-wide barrier and read by every block after it, so the whole grid learns that the
// peers' gradients may be incomplete and leaves without touching parameters or optimizer state.
__device__ unsigned int g_abort_epoch = 0xFFFFFFFFu;

// flag exchange among ranks, executed by the first `world` threads of block 0
__device__ bool exchange(const Args& a, int phase) {
  bool ok = true;
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    st_release_sys(a.flags[peer] + phase * MAX_RANKS + a.rank, a.epoch);
    const uint32_t* mine = a.flags[a.rank] + phase * MAX_RANKS + peer;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(mine) - a.epoch) < 0) {
      if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
        *(volatile int*)a.status = 0x300 + phase;
        if (phase == 0) atomicExch(&g_abort_epoch, a.epoch);
        __threadfence_system();
        ok = false;
        break;
      }
    }
  }
  return ok;
}

// One thread handles U 16-byte pieces per trip and issues ALL its peer loads of the trip (every
// rank, every piece: W * U = 16 loads of 16 bytes) before it adds anything, so 256 bytes per thread
// are in flight on NVLink at any time.  A peer load takes a few microseconds: with one load in
// flight per thread the links ran at well under half their rate, and with the ranks visited one
// after the other each trip paid the latency once per rank.  The sum still runs in rank order, so
// every rank computes bitwise the same value.
template <int KIND>
__device__ __forceinline__ void update_piece(const Args& a, long long i, float4 gv, float inv) {
  gv.x *= inv; gv.y *= inv; gv.z *= inv; gv.w *= inv;
  float4 p = *reinterpret_cast<const float4*>(a.param[a.rank] + i);
  const long long li = i - a.lo;
  float4 s1 = make_float4(0, 0, 0, 0), s2 = make_float4(0, 0, 0, 0);
  if (KIND >= 1) s1 = *reinterpret_cast<const float4*>(a.slot1 + li);
  if (KIND == 4) s2 = *reinterpret_cast<const float4*>(a.slot2 + li);
  opt_one<KIND>(p.x, gv.x, s1.x, s2.x, a.h);
  opt_one<KIND>(p.y, gv.y, s1.y, s2.y, a.h);
  opt_one<KIND>(p.z, gv.z, s1.z, s2.z, a.h);
  opt_one<KIND>(p.w, gv.w, s1.w, s2.w, a.h);
  if (KIND >= 1) *reinterpret_cast<float4*>(a.slot1 + li) = s1;
  if (KIND == 4) *reinterpret_cast<float4*>(a.slot2 + li) = s2;
  if (a.param_mc) {
    multimem_st(a.param_mc + i, p);
  } else {
#pragma unroll 1
    for (int r = 0; r < a.world; ++r) st_peer(a.param[r] + i, p);
  }
}

// W = number of ranks when it is 2, 4 or 8 (all loads of a trip in flight), 0 = any (rank by rank)
template <int KIND, int W>
__device__ void reduce_update_shard_w(const Args& a, long long tid, long long nthreads) {
  constexpr int U = W ? 16 / W : 8;
  const float inv = 1.f / (float)a.world;
  const long long lo4 = a.lo >> 2, hi4 = a.hi >> 2;
  for (long long base = lo4 + tid; base < hi4; base += nthreads * U) {
    float4 g[U];
    if (a.grad_mc) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i4 = base + u * nthreads;
        g[u] = i4 < hi4 ? multimem_ld_reduce(a.grad_mc + (i4 << 2)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else if (W) {
      float4 v[W ? W : 1][U];
#pragma unroll
      for (int r = 0; r < W; ++r) {
        const float* src = a.grad[r];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i4 = base + u * nthreads;
          v[r][u] = i4 < hi4 ? ld_peer(src + (i4 << 2)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        g[u] = v[0][u];
#pragma unroll
        for (int r = 1; r < W; ++r) { g[u].x += v[r][u].x; g[u].y += v[r][u].y; g[u].z += v[r][u].z; g[u].w += v[r][u].w; }
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) g[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
      for (int r = 0; r < a.world; ++r) {       // fixed order: bitwise identical on every rank
        const float* src = a.grad[r];
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i4 = base + u * nthreads;
          v[u] = i4 < hi4 ? ld_peer(src + (i4 << 2)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) { g[u].x += v[u].x; g[u].y += v[u].y; g[u].z += v[u].z; g[u].w += v[u].w; }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i4 = base + u * nthreads;
      if (i4 < hi4) update_piece<KIND>(a, i4 << 2, g[u], inv);
    }
  }
}

template <int KIND>
__device__ void reduce_update_shard(const Args& a, long long tid, long long nthreads) {
  if (a.world == 2) reduce_update_shard_w<KIND, 2>(a, tid, nthreads);
  else if (a.world == 4) reduce_update_shard_w<KIND, 4>(a, tid, nthreads);
  else if (a.world == 8) reduce_update_shard_w<KIND, 8>(a, tid, nthreads);
  else reduce_update_shard_w<KIND, 0>(a, tid, nthreads);
}

template <int KIND>
__global__ void __launch_bounds__(512, 1) fused_allreduce_update(const Args a) {
  cg::grid_group grid = cg::this_grid();
  exchange(a, 0);                          // gradients of every rank are complete
  grid.sync();
  // a peer never signalled: its gradients may be incomplete, so nothing is reduced, no parameter or
  // optimizer slot is written and no shard is published (every thread of the grid takes this exit)
  if (*(volatile unsigned int*)&g_abort_epoch == a.epoch) return;
  reduce_update_shard<KIND>(a, blockIdx.x * (long long)blockDim.x + threadIdx.x,
                            (long long)gridDim.x * blockDim.x);
  __threadfence_system();
  grid.sync();
  exchange(a, 1);                          // every shard has been written to every rank
}

// Single-GPU stand-in used by tests: all "ranks" live in one device's memory and
// their shards are processed one after the other by one launch (no flags, no
// cross-kernel waiting).
template <int KIND>
__global__ void emulate_all_ranks(Args a, long long shard) {
  for (int r = 0; r < a.world; ++r) {
    Args b = a;
    b.rank = r;
    b.lo = r * shard;
    b.hi = (r == a.world - 1) ? a.n : (r + 1) * shard;
    b.slot1 = a.slot1 ? a.slot1 + b.lo : nullptr;     // emulation keeps the state shards in one array
    b.slot2 = a.slot2 ? a.slot2 + b.lo : nullptr;
    reduce_update_shard<KIND>(b, blockIdx.x * (long long)blockDim.x + threadIdx.x,
                              (long long)gridDim.x * blockDim.x);
  }
}

int* g_status_host = nullptr;
int* g_status_dev[64] = {nullptr};
int* status_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (!g_status_host) {
    if (cudaHostAlloc(reinterpret_cast<void**>(&g_status_host), 64 * sizeof(int),
                      cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess)
      return nullptr;
    for (int i = 0; i < 64; ++i) g_status_host[i] = 0;
  }
  if (!g_status_dev[dev]) {
    int* d = nullptr;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), g_status_host, 0) != cudaSuccess) return nullptr;
    g_status_dev[dev] = d + dev;
  }
  return g_status_dev[dev];
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int KIND>
int launch(const Args& a, int blocks, cudaStream_t st) {
  void* params[] = {const_cast<Args*>(&a)};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(fused_allreduce_update<KIND>), dim3(blocks),
                                              dim3(512), params, 0, st);
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

void fill(Args& a, int kind, int rank, int world, void* const* grad, void* const* param, void* const* flags,
          const void* grad_mc, void* param_mc, float* slot1, float* slot2, long long n, const float* hyper,
          uint32_t epoch) {
  for (int r = 0; r < MAX_RANKS; ++r) {
    a.grad[r] = r < world ? static_cast<const float*>(grad[r]) : nullptr;
    a.param[r] = r < world ? static_cast<float*>(param[r]) : nullptr;
    a.flags[r] = (flags && r < world) ? static_cast<uint32_t*>(flags[r]) : nullptr;
  }
  a.grad_mc = static_cast<const float*>(grad_mc);
  a.param_mc = static_cast<float*>(param_mc);
  a.slot1 = slot1; a.slot2 = slot2; a.n = n; a.rank = rank; a.world = world; a.kind = kind; a.epoch = epoch;
  for (int i = 0; i < 8; ++i) a.h[i] = hyper[i];
  const long long per = ((n / 4 + world - 1) / world) * 4;     // shard size, multiple of 4 floats
  a.lo = per * rank < n ? per * rank : n;
  a.hi = (per * (rank + 1) < n && rank != world - 1) ? per * (rank + 1) : n;
  if (a.lo > a.hi) a.lo = a.hi;
}

}  // namespace

extern "C" {

// Elements of the shard owned by `rank` (callers size the sharded optimizer state with it).
long long tsb_fused_shard_elems(long long n, int rank, int world) {
  const long long per = ((n / 4 + world - 1) / world) * 4;
  long long lo = per * rank < n ? per * rank : n;
  long long hi = (per * (rank + 1) < n && rank != world - 1) ? per * (rank + 1) : n;
  return hi > lo ? hi - lo : 0;
}
long long tsb_fused_shard_begin(long long n, int rank, int world) {
  const long long per = ((n / 4 + world - 1) / world) * 4;
  return per * rank < n ? per * rank : n;
}

// grad / param / flags: arrays of `world` peer pointers (index = rank).  flags point to 2*16 uint32 words
// per rank, zero-initialised once; epoch must increase by one per call on every rank (calls that may be in
// flight together, e.g. one per bucket, need flag words of their own).  max_blocks > 0 caps the grid.
int tsb_fused_allreduce_update(int kind, int rank, int world, void* const* grad, void* const* param,
                               void* const* flags, const void* grad_mc, void* param_mc, float* slot1,
                               float* slot2, long long n, const float* hyper, unsigned int epoch, int max_blocks,
                               void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || kind < 0 || kind > 4 || n <= 0 || (n & 3))
    return TSB_ERR_ARG;
  Args a;
  fill(a, kind, rank, world, grad, param, flags, grad_mc, param_mc, slot1, slot2, n, hyper, epoch);
  a.status = status_word();
  if (!a.status) return TSB_ERR_LAUNCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long want = ((a.hi - a.lo) / 4 + 511) / 512;
  int blocks = (int)(want < 1 ? 1 : (want > sm_count() ? sm_count() : want));
  if (max_blocks > 0 && blocks > max_blocks) blocks = max_blocks;     // leave SMs to the kernels it overlaps with
  int rc;
  switch (kind) {
    case 0: rc = launch<0>(a, blocks, st); break;
    case 1: rc = launch<1>(a, blocks, st); break;
    case 2: rc = launch<2>(a, blocks, st); break;
    case 3: rc = launch<3>(a, blocks, st); break;
    default: rc = launch<4>(a, blocks, st); break;
  }
  if (rc) return rc;
  int dev = 0;
  cudaGetDevice(&dev);
  const int late = g_status_host ? *(volatile int*)(g_status_host + dev) : 0;
  return late ? (TSB_ERR_TIMEOUT | (late << 8)) : TSB_OK;
}

// One-GPU emulation of all ranks (tests): grad[r] / param[r] are plain device pointers of one device,
// slot1 / slot2 hold the full-length state.
int tsb_fused_allreduce_emulate(int kind, int world, void* const* grad, void* const* param, float* slot1,
                                float* slot2, long long n, const float* hyper, void* stream) {
  if (world < 1 || world > MAX_RANKS || kind < 0 || kind > 4 || n <= 0 || (n & 3)) return TSB_ERR_ARG;
  Args a;
  fill(a, kind, 0, world, grad, param, nullptr, nullptr, nullptr, slot1, slot2, n, hyper, 1);
  a.status = nullptr;
  const long long shard = ((n / 4 + world - 1) / world) * 4;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (kind) {
    case 0: emulate_all_ranks<0><<<sm_count(), 512, 0, st>>>(a, shard); break;
    case 1: emulate_all_ranks<1><<<sm_count(), 512, 0, st>>>(a, shard); break;
    case 2: emulate_all_ranks<2><<<sm_count(), 512, 0, st>>>(a, shard); break;
    case 3: emulate_all_ranks<3><<<sm_count(), 512, 0, st>>>(a, shard); break;
    default: emulate_all_ranks<4><<<sm_count(), 512, 0, st>>>(a, shard); break;
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

// Synchronise and return (then clear) the status word: 0 = clean.
int tsb_comm_status(void* stream) {
  cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  int dev = 0;
  cudaGetDevice(&dev);
  if (!g_status_host) return 0;
  const int v = *(volatile int*)(g_status_host + dev);
  g_status_host[dev] = 0;
  return v;
}

}  // extern "C"
