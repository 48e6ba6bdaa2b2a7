// One-hot, embedding lookup (+ scatter-add gradient), counter-based dropout,
// CSR sparse x dense products, and the multi-tensor optimizer step.
//
// Roles in the reference: src/ops/OneHot.cu, EmbeddingLookup.cu (which ignores
// the ids; this one honours them), CudnnDropout.cu, CuSparseCsrmv.cu /
// CuSparseCsrmm.cu (legacy cuSPARSE) and Optimizers.cu:3-149 (one launch per
// parameter tensor there, one launch per 64 tensors here).
#include <cuda_runtime.h>
#include <stdint.h>

#define TSB_OK 0
#define TSB_ERR_ARG 1
#define TSB_ERR_LAUNCH 3

namespace {

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
int ew_grid(long long work) {
  long long blocks = (work + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}
int done() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

__global__ void one_hot_kernel(const float* __restrict__ idx, float* __restrict__ y, long long n, long long k) {
  const long long total = n * k;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / k, c = i - r * k;
    y[i] = ((long long)idx[r] == c) ? 1.f : 0.f;
  }
}

// Rows that are a multiple of four classes long: one block row-slice per row, 16-byte stores, no division
// per element (grid.y walks the rows, grid.x * blockDim.x the 4-class groups of a row).
__global__ void one_hot_rows_v4(const float* __restrict__ idx, float4* __restrict__ y, long long n, int k4) {
  for (long long r = blockIdx.y; r < n; r += gridDim.y) {
    const long long id = (long long)idx[r];
    float4* yr = y + r * k4;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < k4; c += gridDim.x * blockDim.x) {
      const long long c0 = 4ll * c;
      yr[c] = make_float4(id == c0 ? 1.f : 0.f, id == c0 + 1 ? 1.f : 0.f, id == c0 + 2 ? 1.f : 0.f,
                          id == c0 + 3 ? 1.f : 0.f);
    }
  }
}

__global__ void embedding_kernel(const float* __restrict__ table, const float* __restrict__ idx,
                                 float* __restrict__ y, long long n, long long vocab, long long dim) {
  const long long total = n * dim;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / dim, c = i - r * dim;
    long long id = (long long)idx[r];
    y[i] = (id >= 0 && id < vocab) ? table[id * dim + c] : 0.f;
  }
}

__global__ void embedding_grad_kernel(const float* __restrict__ g, const float* __restrict__ idx,
                                      float* __restrict__ dtable, long long n, long long vocab, long long dim) {
  const long long total = n * dim;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / dim, c = i - r * dim;
    long long id = (long long)idx[r];
    if (id >= 0 && id < vocab) atomicAdd(dtable + id * dim + c, g[i]);
  }
}

// splitmix64 of (seed, element index): the keep decision is a pure function of both
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long i) {
  unsigned long long x = i + seed * 0x9E3779B97F4A7C15ull;
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return (float)(x >> 40) * (1.0f / 16777216.0f);
}

// step_dev (may be null): index of the training step, kept on the device by the executor so that a
// step replayed from a CUDA graph still draws a new mask; the seed is mixed exactly as on the host.
// offset: index of x[0] in the whole tensor when x is a batch piece of it (the mask is a function of the
// element's index in the WHOLE tensor, so a tensor computed piece by piece gets the same mask).
__global__ void dropout_kernel(const float* __restrict__ x, float* __restrict__ y, long long n, float keep,
                               unsigned long long seed, const unsigned long long* __restrict__ step_dev,
                               unsigned long long offset) {
  if (step_dev) seed = (seed + 0x632BE5ABull * *step_dev) & 0x7FFFFFFFFFFFFFFFull;
  const float inv = 1.f / keep;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    y[i] = uniform01(seed, (unsigned long long)i + offset) < keep ? x[i] * inv : 0.f;
}

// out[r, :] = sum_j vals[j] * dense[col[j], :]   (one warp per sparse row)
__global__ void csrmm_kernel(const float* __restrict__ vals, const float* __restrict__ rowptr,
                             const float* __restrict__ colidx, long long nrow, const float* __restrict__ dense,
                             float* __restrict__ out, long long ncols) {
  const int lane = threadIdx.x & 31;
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (row >= nrow) return;
  const long long b = (long long)rowptr[row], e = (long long)rowptr[row + 1];
  for (long long c = lane; c < ncols; c += 32) {
    float acc = 0.f;
    for (long long j = b; j < e; ++j) acc += vals[j] * dense[(long long)colidx[j] * ncols + c];
    out[row * ncols + c] = acc;
  }
}
// out[col[j], :] += vals[j] * dense[r, :]   (transposed sparse operand; out pre-zeroed)
__global__ void csrmm_t_kernel(const float* __restrict__ vals, const float* __restrict__ rowptr,
                               const float* __restrict__ colidx, long long nrow, const float* __restrict__ dense,
                               float* __restrict__ out, long long ncols) {
  const int lane = threadIdx.x & 31;
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (row >= nrow) return;
  const long long b = (long long)rowptr[row], e = (long long)rowptr[row + 1];
  for (long long j = b; j < e; ++j) {
    const float v = vals[j];
    const long long oc = (long long)colidx[j];
    for (long long c = lane; c < ncols; c += 32) atomicAdd(out + oc * ncols + c, v * dense[row * ncols + c]);
  }
}
__global__ void zero_kernel(float* __restrict__ y, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    y[i] = 0.f;
}

// ------------------------------------------------------------------ optimizers
constexpr int MAX_TENSORS = 64;
struct OptArgs {
  float* p[MAX_TENSORS];
  const float* g[MAX_TENSORS];
  float* s1[MAX_TENSORS];
  float* s2[MAX_TENSORS];
  long long n[MAX_TENSORS];
  float h[8];
  const float* hdev;     // Adam only, may be null: {beta1^t, beta2^t} kept on the device (see tsb_adam_advance)
  int count;
};

template <int KIND>
__device__ __forceinline__ void opt_one(float& p, float g, float& s1, float& s2, const float* h) {
  if (KIND == 0) {                // sgd: h = {lr}
    p -= h[0] * g;
  } else if (KIND == 1) {         // momentum: h = {lr, momentum}
    s1 = h[1] * s1 - h[0] * g;
    p += s1;
  } else if (KIND == 2) {         // nesterov
    const float lr_g = -h[0] * g;
    s1 = h[1] * (s1 + lr_g);
    p += s1 + lr_g;
  } else if (KIND == 3) {         // adagrad: h = {lr, eps}
    s1 += g * g;
    p -= h[0] * g / (sqrtf(s1) + h[1]);
  } else {                        // adam: h = {lr, b1, b2, b1^t, b2^t, eps}
    s1 = h[1] * s1 + (1.f - h[1]) * g;
    s2 = h[2] * s2 + (1.f - h[2]) * g * g;
    const float mc = s1 / (1.f - h[3]);
    const float vc = s2 / (1.f - h[4]);
    p -= h[0] * mc / (sqrtf(vc) + h[5]);
  }
}

template <int KIND>
__global__ void opt_kernel(const OptArgs a) {
  const int t = blockIdx.y;
  if (t >= a.count) return;
  float hloc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) hloc[i] = a.h[i];
  if (KIND == 4 && a.hdev) { hloc[3] = a.hdev[0]; hloc[4] = a.hdev[1]; }
  float* p = a.p[t];
  const float* g = a.g[t];
  float* s1 = a.s1[t];
  float* s2 = a.s2[t];
  const long long n = a.n[t];
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  // 16 bytes per access when every array of this tensor is 16-byte aligned; scalar tail / fallback
  const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                     (KIND >= 1 ? reinterpret_cast<uintptr_t>(s1) : 0) |
                     (KIND == 4 ? reinterpret_cast<uintptr_t>(s2) : 0)) & 15) == 0;
  const long long n4 = vec ? n / 4 : 0;
  for (long long i = tid; i < n4; i += nthreads) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    float4 v1 = make_float4(0, 0, 0, 0), v2 = make_float4(0, 0, 0, 0);
    if (KIND >= 1) v1 = reinterpret_cast<float4*>(s1)[i];
    if (KIND == 4) v2 = reinterpret_cast<float4*>(s2)[i];
    opt_one<KIND>(pv.x, gv.x, v1.x, v2.x, hloc);
    opt_one<KIND>(pv.y, gv.y, v1.y, v2.y, hloc);
    opt_one<KIND>(pv.z, gv.z, v1.z, v2.z, hloc);
    opt_one<KIND>(pv.w, gv.w, v1.w, v2.w, hloc);
    reinterpret_cast<float4*>(p)[i] = pv;
    if (KIND >= 1) reinterpret_cast<float4*>(s1)[i] = v1;
    if (KIND == 4) reinterpret_cast<float4*>(s2)[i] = v2;
  }
  for (long long i = n4 * 4 + tid; i < n; i += nthreads) {
    float pv = p[i], v1 = (KIND >= 1) ? s1[i] : 0.f, v2 = (KIND == 4) ? s2[i] : 0.f;
    opt_one<KIND>(pv, g[i], v1, v2, hloc);
    p[i] = pv;
    if (KIND >= 1) s1[i] = v1;
    if (KIND == 4) s2[i] = v2;
  }
}

// Adam's bias-correction powers live on the device so that a captured step (CUDA graph) advances
// them by itself: one thread multiplies {beta1^t, beta2^t} by {beta1, beta2} before the update.
__global__ void step_advance_kernel(unsigned long long* step_dev) { *step_dev += 1ull; }

__global__ void adam_advance_kernel(float* hdev, float b1, float b2) {
  hdev[0] *= b1;
  hdev[1] *= b2;
}

}  // namespace

extern "C" {

int tsb_adam_advance(float* hdev, float b1, float b2, void* stream) {
  if (!hdev) return TSB_ERR_ARG;
  adam_advance_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(hdev, b1, b2);
  return done();
}

int tsb_one_hot(const float* idx, float* y, long long n, long long k, void* stream) {
  if (n <= 0 || k <= 0) return TSB_ERR_ARG;
  if ((k & 3) == 0 && k / 4 < (1ll << 30) && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
    const int k4 = (int)(k / 4);
    int gx = (k4 + 255) / 256;
    if (gx > 32) gx = 32;
    long long gy = n < 65535 ? n : 65535;
    one_hot_rows_v4<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        idx, reinterpret_cast<float4*>(y), n, k4);
    return done();
  }
  one_hot_kernel<<<ew_grid(n * k), 256, 0, static_cast<cudaStream_t>(stream)>>>(idx, y, n, k);
  return done();
}

int tsb_embedding(const float* table, const float* idx, float* y, long long n, long long vocab, long long dim,
                  void* stream) {
  if (n <= 0) return TSB_OK;
  embedding_kernel<<<ew_grid(n * dim), 256, 0, static_cast<cudaStream_t>(stream)>>>(table, idx, y, n, vocab, dim);
  return done();
}

int tsb_embedding_grad(const float* g, const float* idx, float* dtable, long long n, long long vocab,
                       long long dim, void* stream) {
  if (n <= 0) return TSB_OK;
  embedding_grad_kernel<<<ew_grid(n * dim), 256, 0, static_cast<cudaStream_t>(stream)>>>(g, idx, dtable, n, vocab,
                                                                                         dim);
  return done();
}

int tsb_dropout(const float* x, float* y, long long n, float keep, unsigned long long seed,
                const unsigned long long* step_dev, unsigned long long offset, void* stream) {
  if (n <= 0) return TSB_OK;
  if (!(keep > 0.f)) return TSB_ERR_ARG;
  dropout_kernel<<<ew_grid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, n, keep, seed, step_dev, offset);
  return done();
}

// ++*step_dev on the stream (one thread): the executor's step counter, advanced at the start of a step
int tsb_step_advance(unsigned long long* step_dev, void* stream) {
  if (!step_dev) return TSB_ERR_ARG;
  step_advance_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(step_dev);
  return done();
}

int tsb_csrmm(const float* vals, const float* rowptr, const float* colidx, long long nrow, long long ncol,
              const float* dense, float* out, int trans_a, long long ncols_dense, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (nrow <= 0 || ncols_dense <= 0) return TSB_ERR_ARG;
  const long long threads = nrow * 32;
  if (!trans_a) {
    csrmm_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(vals, rowptr, colidx, nrow, dense, out,
                                                                     ncols_dense);
  } else {
    zero_kernel<<<ew_grid(ncol * ncols_dense), 256, 0, st>>>(out, ncol * ncols_dense);
    csrmm_t_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(vals, rowptr, colidx, nrow, dense, out,
                                                                       ncols_dense);
  }
  return done();
}

int tsb_optimizer_step_dev(int kind, int count, float** params, const float** grads, float** slot1, float** slot2,
                           const long long* sizes, const float* hyper, const float* hyper_dev, void* stream);

int tsb_optimizer_step(int kind, int count, float** params, const float** grads, float** slot1, float** slot2,
                       const long long* sizes, const float* hyper, void* stream) {
  return tsb_optimizer_step_dev(kind, count, params, grads, slot1, slot2, sizes, hyper, nullptr, stream);
}

// hyper_dev (Adam, optional): device array {beta1^t, beta2^t} that overrides hyper[3], hyper[4]
int tsb_optimizer_step_dev(int kind, int count, float** params, const float** grads, float** slot1, float** slot2,
                           const long long* sizes, const float* hyper, const float* hyper_dev, void* stream) {
  if (count <= 0 || count > MAX_TENSORS || kind < 0 || kind > 4) return TSB_ERR_ARG;
  OptArgs a;
  a.count = count;
  a.hdev = hyper_dev;
  long long biggest = 0;
  for (int i = 0; i < count; ++i) {
    a.p[i] = params[i]; a.g[i] = grads[i];
    a.s1[i] = slot1 ? slot1[i] : nullptr;
    a.s2[i] = slot2 ? slot2[i] : nullptr;
    a.n[i] = sizes[i];
    if (sizes[i] > biggest) biggest = sizes[i];
    if (kind >= 1 && !a.s1[i]) return TSB_ERR_ARG;
    if (kind == 4 && !a.s2[i]) return TSB_ERR_ARG;
  }
  for (int i = 0; i < 8; ++i) a.h[i] = hyper[i];
  long long bx = (biggest / 4 + 255) / 256;
  if (bx > 8 * sm_count()) bx = 8 * sm_count();
  if (bx < 1) bx = 1;
  dim3 grid((unsigned)bx, count);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (kind) {
    case 0: opt_kernel<0><<<grid, 256, 0, st>>>(a); break;
    case 1: opt_kernel<1><<<grid, 256, 0, st>>>(a); break;
    case 2: opt_kernel<2><<<grid, 256, 0, st>>>(a); break;
    case 3: opt_kernel<3><<<grid, 256, 0, st>>>(a); break;
    default: opt_kernel<4><<<grid, 256, 0, st>>>(a); break;
  }
  return done();
}

}  // extern "C"
