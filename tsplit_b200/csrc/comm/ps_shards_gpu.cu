// GPU-resident parameter-server shards on one NVLink / NVSwitch box.
//
// The reference's parameter server (vendored ps-lite, src/ps/worker.cc:108-133) keeps the weights on
// server processes: a worker pushes delta = -lr / workers * gradient, the server adds it to the key's
// value, the worker pulls the value back; BSP puts a barrier between push and pull, ASP does not.
// On one box every GPU is both a worker and a server: the key space is one flat array in symmetric
// (peer-mapped) memory and rank r serves the r-th slice of it.
//
//   BSP  push + barrier + pull of every worker = all-reduce of the deltas applied to the served slice
//        and broadcast: that is tsb_fused_allreduce_update with the plain-SGD rule (fused_allreduce.cu).
//   ASP  this file: ONE kernel per worker that (1) adds its delta slice by slice into the serving rank's
//        memory with red.add over NVLink and (2) reads every slice back into the worker's local copy,
//        taking whatever the other workers have pushed by then.  No flag, no wait on a peer: a worker
//        that is late or gone only means its deltas are not in the values the others read.
//
// Peer memory is touched with plain red / ld on generic addresses only (no TMA, no multicast).
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cg = cooperative_groups;

#define TSB_OK 0
#define TSB_ERR_ARG 1
#define TSB_ERR_LAUNCH 3

namespace {

constexpr int MAX_RANKS = 16;

struct PsArgs {
  float* served[MAX_RANKS];   // peer pointers to the key array; rank r serves [r * per, (r + 1) * per)
  const float* delta;         // this worker's update (gradient), full length
  float* local;               // this worker's copy of the values, full length
  long long n, per;
  int world;
  float scale;                // delta is multiplied by this before it is pushed (-lr / workers)
};

__device__ __forceinline__ void red_add_peer(float* p, float v) {
  asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ float4 ld_peer(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(512, 1) ps_asp_push_pull(const PsArgs a) {
  cg::grid_group grid = cg::this_grid();
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  // push: every element goes to the rank that serves it
  for (long long i = tid * 4; i < a.n; i += nth * 4) {
    const int owner = (int)(i / a.per);
    const float4 d = *reinterpret_cast<const float4*>(a.delta + i);
    float* dst = a.served[owner] + i;
    red_add_peer(dst + 0, d.x * a.scale);
    red_add_peer(dst + 1, d.y * a.scale);
    red_add_peer(dst + 2, d.z * a.scale);
    red_add_peer(dst + 3, d.w * a.scale);
  }
  __threadfence_system();
  grid.sync();                 // this worker's own pushes are out before it pulls
  // pull: read every slice from its server
  for (long long i = tid * 4; i < a.n; i += nth * 4) {
    const int owner = (int)(i / a.per);
    *reinterpret_cast<float4*>(a.local + i) = ld_peer(a.served[owner] + i);
  }
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

}  // namespace

extern "C" {

// Elements served by one rank (a multiple of 4; the last rank's slice may be shorter).
long long tsb_ps_gpu_slice(long long n, int world) { return ((n / 4 + world - 1) / world) * 4; }

// ASP push + pull of one worker.  served: `world` peer pointers to the key array (index = serving rank),
// delta / local: this worker's device arrays of n floats (n a multiple of 4, all 16-byte aligned).
int tsb_ps_gpu_asp(void* const* served, const float* delta, float* local, long long n, int world, float scale,
                   void* stream) {
  if (world < 1 || world > MAX_RANKS || n <= 0 || (n & 3) || !delta || !local) return TSB_ERR_ARG;
  PsArgs a;
  for (int r = 0; r < MAX_RANKS; ++r) a.served[r] = r < world ? static_cast<float*>(served[r]) : nullptr;
  a.delta = delta; a.local = local; a.n = n; a.world = world; a.scale = scale;
  a.per = tsb_ps_gpu_slice(n, world);
  long long want = (n / 4 + 511) / 512;
  const int blocks = (int)(want < 1 ? 1 : (want > sm_count() ? sm_count() : want));
  void* params[] = {&a};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ps_asp_push_pull), dim3(blocks), dim3(512),
                                              params, 0, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

}  // extern "C"
