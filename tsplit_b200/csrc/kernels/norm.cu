// Batch normalisation (training mode, channels-last [rows, C] view with a row
// stride) and layer normalisation, fp32.
//
// Batch norm forward = column statistics (two-stage, fixed order, combined in
// double) + one fused normalise/scale/shift(/ReLU) pass; backward = one column
// reduction (sum dy, sum dy*xhat) + one fused dx pass.  All passes read/write
// 16 bytes per thread and are HBM-bound by construction: x is read twice and y
// written once in forward; dy and x are read twice and dx written once in
// backward.  The statistics / apply stages are also exported separately so a
// micro-tensor executor can accumulate statistics over batch pieces.
//
// Role in the reference: cudnnBatchNormalizationForwardTraining / Backward
// (src/ops/CudnnBn.cu:12-382).
#include <cuda_runtime.h>
#include <stdint.h>

#include "norm_static.h"
#include "scratch.h"

#define TSB_OK 0
#define TSB_ERR_ARG 1
#define TSB_ERR_UNSUPPORTED 2
#define TSB_ERR_LAUNCH 3
#define TSB_ERR_OOM 5
#define TSB_ERR_SCRATCH 7

namespace {

constexpr int MAX_CHUNKS = 128;
constexpr long long PLANE_FLOATS = (long long)MAX_CHUNKS * 8192;   // one partial plane: chunks x channels
constexpr long long SCRATCH_FLOATS = 2 * PLANE_FLOATS;              // two planes (up to 8192 channels at MAX_CHUNKS)

float* scratch() {
  return static_cast<float*>(tsb_scratch::get(nullptr, tsb_scratch::NORM_PARTIALS, SCRATCH_FLOATS * sizeof(float)));
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

int done() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

// Column partial sums over a chunk of rows.  A block of 256 threads covers `cw` float4 columns
// (cw = min(32, C/4)) with 256/cw row lanes, so narrow tensors (64 channels) still keep every
// thread busy; each thread has four independent rows in flight.
// MODE 0: p0 = sum x, p1 = sum x^2.   MODE 1: p0 = sum dy, p1 = sum dy * (x - mean) * invstd.
// `rscale` / `rbias` (MODE 1 only, may be null): scale and shift of a fused BN+ReLU forward; dy then
// counts only where the forward output (x - mean) * invstd * scale + bias was positive.  The sign is
// recomputed from x, which this pass reads anyway, instead of reading the forward output.
constexpr int STAT_THREADS = 256;
constexpr int STAT_UNROLL = 4;

__device__ __forceinline__ void stat_accum0(float4& a0, float4& a1, const float4 v) {
  a0.x += v.x; a0.y += v.y; a0.z += v.z; a0.w += v.w;
  a1.x += v.x * v.x; a1.y += v.y * v.y; a1.z += v.z * v.z; a1.w += v.w * v.w;
}
__device__ __forceinline__ void stat_accum1(float4& a0, float4& a1, float4 g, const float4 x, const float4 mu,
                                            const float4 is) {
  a0.x += g.x; a0.y += g.y; a0.z += g.z; a0.w += g.w;
  a1.x += g.x * (x.x - mu.x) * is.x; a1.y += g.y * (x.y - mu.y) * is.y;
  a1.z += g.z * (x.z - mu.z) * is.z; a1.w += g.w * (x.w - mu.w) * is.w;
}
// dy where the fused forward output was positive, else 0 (same expression as bn_apply_fwd)
__device__ __forceinline__ float4 relu_mask(float4 g, const float4 x, const float4 mu, const float4 is,
                                            const float4 sc, const float4 bi) {
  g.x = ((x.x - mu.x) * is.x * sc.x + bi.x) > 0.f ? g.x : 0.f;
  g.y = ((x.y - mu.y) * is.y * sc.y + bi.y) > 0.f ? g.y : 0.f;
  g.z = ((x.z - mu.z) * is.z * sc.z + bi.z) > 0.f ? g.z : 0.f;
  g.w = ((x.w - mu.w) * is.w * sc.w + bi.w) > 0.f ? g.w : 0.f;
  return g;
}

template <int MODE>
__global__ void __launch_bounds__(STAT_THREADS)
col_partial(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ mean,
            const float* __restrict__ invstd, float* __restrict__ part, long long rows, int C,
            long long lda, long long ldb, int chunks, int cw, const float* __restrict__ rscale = nullptr,
            const float* __restrict__ rbias = nullptr, long long plane = PLANE_FLOATS) {
  __shared__ float4 s0[STAT_THREADS], s1[STAT_THREADS];
  const int rl = STAT_THREADS / cw;               // row lanes
  const int cx = threadIdx.x % cw, ry = threadIdx.x / cw;
  const int c = (blockIdx.x * cw + cx) * 4;
  const int ch = blockIdx.y;
  const long long per = (rows + chunks - 1) / chunks;
  const long long r0 = ch * per, r1 = min(rows, r0 + per);
  float4 acc0 = make_float4(0, 0, 0, 0), acc1 = make_float4(0, 0, 0, 0);
  const bool active = ry < rl && c < C;
  if (active) {
    float4 mu = make_float4(0, 0, 0, 0), is = make_float4(1, 1, 1, 1);
    float4 sc = make_float4(0, 0, 0, 0), bi = make_float4(0, 0, 0, 0);
    const bool relu = MODE == 1 && rscale != nullptr;
    if (MODE == 1) {
      mu = *reinterpret_cast<const float4*>(mean + c);
      is = *reinterpret_cast<const float4*>(invstd + c);
      if (relu) {
        sc = *reinterpret_cast<const float4*>(rscale + c);
        bi = *reinterpret_cast<const float4*>(rbias + c);
      }
    }
    long long r = r0 + ry;
    for (; r + (STAT_UNROLL - 1) * rl < r1; r += STAT_UNROLL * rl) {
      float4 v[STAT_UNROLL], x[STAT_UNROLL];
#pragma unroll
      for (int u = 0; u < STAT_UNROLL; ++u) {
        v[u] = *reinterpret_cast<const float4*>(a + (r + u * rl) * lda + c);
        if (MODE == 1) x[u] = *reinterpret_cast<const float4*>(b + (r + u * rl) * ldb + c);
      }
#pragma unroll
      for (int u = 0; u < STAT_UNROLL; ++u) {
        if (MODE == 0) {
          stat_accum0(acc0, acc1, v[u]);
        } else {
          if (relu) v[u] = relu_mask(v[u], x[u], mu, is, sc, bi);
          stat_accum1(acc0, acc1, v[u], x[u], mu, is);
        }
      }
    }
    for (; r < r1; r += rl) {
      float4 v = *reinterpret_cast<const float4*>(a + r * lda + c);
      if (MODE == 0) {
        stat_accum0(acc0, acc1, v);
      } else {
        const float4 xv = *reinterpret_cast<const float4*>(b + r * ldb + c);
        if (relu) v = relu_mask(v, xv, mu, is, sc, bi);
        stat_accum1(acc0, acc1, v, xv, mu, is);
      }
    }
  }
  s0[threadIdx.x] = acc0;
  s1[threadIdx.x] = acc1;
  __syncthreads();
  if (ry == 0 && c < C) {
    float4 t0 = s0[cx], t1 = s1[cx];
    for (int j = 1; j < rl; ++j) {               // fixed order: the result does not depend on scheduling
      const float4 u0 = s0[j * cw + cx], u1 = s1[j * cw + cx];
      t0.x += u0.x; t0.y += u0.y; t0.z += u0.z; t0.w += u0.w;
      t1.x += u1.x; t1.y += u1.y; t1.z += u1.z; t1.w += u1.w;
    }
    float* p0 = part + (long long)ch * C + c;
    float* p1 = part + plane + (long long)ch * C + c;          // second plane
    *reinterpret_cast<float4*>(p0) = t0;
    *reinterpret_cast<float4*>(p1) = t1;
  }
}

// Sum of the chunk partials of one channel, in double and in a fixed order: block = 32 channels
// x FIN_LANES lanes; lane y adds chunks y, y+FIN_LANES, ... (four independent loads in flight),
// lane 0 then adds the lane sums.
constexpr int FIN_LANES = 32;
__device__ __forceinline__ void reduce_partials(const float* __restrict__ part, int chunks, int C, int c,
                                                double& s, double& ss, long long plane = PLANE_FLOATS) {
  __shared__ double sh0[FIN_LANES][33], sh1[FIN_LANES][33];
  double a = 0.0, b = 0.0;
  if (c < C) {
    int ch = threadIdx.y;
    for (; ch + 3 * FIN_LANES < chunks; ch += 4 * FIN_LANES) {
      float x[4], y[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        x[u] = part[(long long)(ch + u * FIN_LANES) * C + c];
        y[u] = part[plane + (long long)(ch + u * FIN_LANES) * C + c];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) { a += x[u]; b += y[u]; }
    }
    for (; ch < chunks; ch += FIN_LANES) {
      a += part[(long long)ch * C + c];
      b += part[plane + (long long)ch * C + c];
    }
  }
  sh0[threadIdx.y][threadIdx.x] = a;
  sh1[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  s = 0.0; ss = 0.0;
  if (threadIdx.y == 0) {
#pragma unroll 8
    for (int j = 0; j < FIN_LANES; ++j) { s += sh0[j][threadIdx.x]; ss += sh1[j][threadIdx.x]; }
  }
}

// Forward finalise: mean / invstd from the partial sums (+ running statistics).  Block (32, FIN_LANES).
__global__ void bn_finalize_fwd(const float* __restrict__ part, int chunks, int C, double count, float eps,
                                float momentum, float* __restrict__ mean, float* __restrict__ invstd,
                                float* __restrict__ run_mean, float* __restrict__ run_var,
                                long long plane = PLANE_FLOATS) {
  const int c = blockIdx.x * 32 + threadIdx.x;
  double s, ss;
  reduce_partials(part, chunks, C, c, s, ss, plane);
  if (threadIdx.y != 0 || c >= C) return;
  const double m = s / count;
  double var = ss / count - m * m;
  if (var < 0.0) var = 0.0;
  mean[c] = (float)m;
  invstd[c] = (float)(1.0 / sqrt(var + (double)eps));
  if (run_mean) {
    run_mean[c] = momentum * run_mean[c] + (1.f - momentum) * (float)m;
    run_var[c] = momentum * run_var[c] + (1.f - momentum) * (float)var;
  }
}

__global__ void bn_finalize_bwd(const float* __restrict__ part, int chunks, int C, float* __restrict__ dscale,
                                float* __restrict__ dbias, long long plane = PLANE_FLOATS) {
  const int c = blockIdx.x * 32 + threadIdx.x;
  double s, ss;
  reduce_partials(part, chunks, C, c, s, ss, plane);
  if (threadIdx.y != 0 || c >= C) return;
  dbias[c] = (float)s;
  dscale[c] = (float)ss;
}

__global__ void bn_apply_fwd(const float* __restrict__ x, const float* __restrict__ scale,
                             const float* __restrict__ bias, const float* __restrict__ mean,
                             const float* __restrict__ invstd, float* __restrict__ y, long long rows, int C,
                             long long ldx, long long ldy, int relu) {
  const int C4 = C >> 2;
  const long long total = rows * C4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / C4;
    const int c = (int)(i - r * C4) * 4;
    const float4 v = *reinterpret_cast<const float4*>(x + r * ldx + c);
    const float4 mu = *reinterpret_cast<const float4*>(mean + c);
    const float4 is = *reinterpret_cast<const float4*>(invstd + c);
    const float4 g = *reinterpret_cast<const float4*>(scale + c);
    const float4 b = *reinterpret_cast<const float4*>(bias + c);
    float4 o;
    o.x = (v.x - mu.x) * is.x * g.x + b.x; o.y = (v.y - mu.y) * is.y * g.y + b.y;
    o.z = (v.z - mu.z) * is.z * g.z + b.z; o.w = (v.w - mu.w) * is.w * g.w + b.w;
    if (relu) { o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f); o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f); }
    *reinterpret_cast<float4*>(y + r * ldy + c) = o;
  }
}

__global__ void bn_apply_bwd(const float* __restrict__ dy, const float* __restrict__ x,
                             const float* __restrict__ scale, const float* __restrict__ mean,
                             const float* __restrict__ invstd, const float* __restrict__ dscale,
                             const float* __restrict__ dbias, float* __restrict__ dx, long long rows, int C,
                             long long lddy, long long ldx, long long lddx, float inv_count,
                             const float* __restrict__ rbias = nullptr) {
  const int C4 = C >> 2;
  const long long total = rows * C4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / C4;
    const int c = (int)(i - r * C4) * 4;
    float4 g = *reinterpret_cast<const float4*>(dy + r * lddy + c);
    const float4 v = *reinterpret_cast<const float4*>(x + r * ldx + c);
    const float4 mu = *reinterpret_cast<const float4*>(mean + c);
    const float4 is = *reinterpret_cast<const float4*>(invstd + c);
    const float4 sc = *reinterpret_cast<const float4*>(scale + c);
    if (rbias) g = relu_mask(g, v, mu, is, sc, *reinterpret_cast<const float4*>(rbias + c));   // fused ReLU
    const float4 ds = *reinterpret_cast<const float4*>(dscale + c);
    const float4 db = *reinterpret_cast<const float4*>(dbias + c);
    float4 o;
    o.x = sc.x * is.x * (g.x - db.x * inv_count - (v.x - mu.x) * is.x * ds.x * inv_count);
    o.y = sc.y * is.y * (g.y - db.y * inv_count - (v.y - mu.y) * is.y * ds.y * inv_count);
    o.z = sc.z * is.z * (g.z - db.z * inv_count - (v.z - mu.z) * is.z * ds.z * inv_count);
    o.w = sc.w * is.w * (g.w - db.w * inv_count - (v.w - mu.w) * is.w * ds.w * inv_count);
    *reinterpret_cast<float4*>(dx + r * lddx + c) = o;
  }
}

// ---- statistics scratch that lives in the library image (see norm_static.h) ----------------
// Two planes of MAX_CHUNKS x 8192 floats (8 MiB), resident on every GPU that loads the library
// until the process exits.  Host code must not hand this name to a kernel: here it is only a
// host-side stand-in, so the device address is looked up once per device.
static __device__ __align__(256) float g_static_stats_scratch[SCRATCH_FLOATS];
float* g_static_scratch_addr[64] = {nullptr};

// Device address of the static scratch on the CURRENT device (looked up on first use).
int static_scratch(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TSB_ERR_ARG;
  if (!g_static_scratch_addr[dev]) {
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_stats_scratch);
    if (e != cudaSuccess || !ptr) return TSB_ERR_LAUNCH | ((int)e << 8);
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return TSB_OK;
}

// Launch geometry of the column statistics: columns per block, row chunks, grid.  Aims at four
// blocks per SM; narrow tensors get more chunks (a plane holds chunks x C partials).
struct StatGeom {
  int cw, chunks;
  dim3 grid;
};
StatGeom stat_geom(long long rows, int C, long long chunk_cap = 1 << 30) {
  StatGeom g;
  const int c4 = C / 4;
  g.cw = c4 < 32 ? c4 : 32;
  const int rl = STAT_THREADS / g.cw;
  const int col_blocks = (c4 + g.cw - 1) / g.cw;
  long long want = (4ll * sm_count() + col_blocks - 1) / col_blocks;
  const long long cap = PLANE_FLOATS / C;
  if (want > cap) want = cap;
  if (want > chunk_cap) want = chunk_cap;
  if (want > 4096) want = 4096;
  const long long by_rows = (rows + (long long)rl * STAT_UNROLL - 1) / ((long long)rl * STAT_UNROLL);
  if (want > by_rows) want = by_rows;
  g.chunks = want < 1 ? 1 : (int)want;
  g.grid = dim3((unsigned)col_blocks, (unsigned)g.chunks);
  return g;
}
inline unsigned fin_blocks(long long C) { return (unsigned)((C + 31) / 32); }

int ew_grid(long long work) {
  long long blocks = (work + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}

// ------------------------------------------------------------------ layer norm (one warp per row)
__global__ void ln_fwd(const float* __restrict__ x, const float* __restrict__ scale, const float* __restrict__ bias,
                       float* __restrict__ y, float* __restrict__ mean, float* __restrict__ invstd, long long rows,
                       int D, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const float* xr = x + row * D;
  float s = 0.f, ss = 0.f;
  for (int i = lane; i < D; i += 32) { const float v = xr[i]; s += v; ss += v * v; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { s += __shfl_xor_sync(0xffffffffu, s, o); ss += __shfl_xor_sync(0xffffffffu, ss, o); }
  const float m = s / D;
  const float var = fmaxf(ss / D - m * m, 0.f);
  const float is = rsqrtf(var + eps);
  if (lane == 0) { mean[row] = m; invstd[row] = is; }
  float* yr = y + row * D;
  for (int i = lane; i < D; i += 32) yr[i] = (xr[i] - m) * is * scale[i] + bias[i];
}

__global__ void ln_bwd_dx(const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ scale,
                          const float* __restrict__ mean, const float* __restrict__ invstd, float* __restrict__ dx,
                          long long rows, int D) {
  const int lane = threadIdx.x & 31;
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const float m = mean[row], is = invstd[row];
  const float* xr = x + row * D;
  const float* gr = dy + row * D;
  float s1 = 0.f, s2 = 0.f;
  for (int i = lane; i < D; i += 32) {
    const float gs = gr[i] * scale[i];
    s1 += gs;
    s2 += gs * (xr[i] - m) * is;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { s1 += __shfl_xor_sync(0xffffffffu, s1, o); s2 += __shfl_xor_sync(0xffffffffu, s2, o); }
  s1 /= D; s2 /= D;
  float* dr = dx + row * D;
  for (int i = lane; i < D; i += 32) dr[i] = is * (gr[i] * scale[i] - s1 - (xr[i] - m) * is * s2);
}

// column sums for dscale / dbias of layer norm: partials over row chunks
__global__ void ln_bwd_params_partial(const float* __restrict__ dy, const float* __restrict__ x,
                                      const float* __restrict__ mean, const float* __restrict__ invstd,
                                      float* __restrict__ part, long long rows, int D, int chunks) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int ch = blockIdx.y;
  if (c >= D) return;
  const long long per = (rows + chunks - 1) / chunks;
  const long long r0 = ch * per, r1 = min(rows, r0 + per);
  float a = 0.f, b = 0.f;
  for (long long r = r0; r < r1; ++r) {
    const float g = dy[r * D + c];
    a += g;
    b += g * (x[r * D + c] - mean[r]) * invstd[r];
  }
  part[(long long)ch * D + c] = a;
  part[PLANE_FLOATS + (long long)ch * D + c] = b;
}

// 16-byte variant (D a multiple of 4): a thread owns four adjacent columns, two rows in flight.
__global__ void ln_bwd_params_partial_v4(const float4* __restrict__ dy, const float4* __restrict__ x,
                                         const float* __restrict__ mean, const float* __restrict__ invstd,
                                         float* __restrict__ part, long long rows, int D4, int chunks) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int ch = blockIdx.y;
  if (c >= D4) return;
  const long long per = (rows + chunks - 1) / chunks;
  const long long r0 = ch * per, r1 = min(rows, r0 + per);
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a, a2 = a, b2 = a;
  long long r = r0;
  for (; r + 1 < r1; r += 2) {
    const float4 g0 = __ldg(dy + r * D4 + c), g1 = __ldg(dy + (r + 1) * D4 + c);
    const float4 v0 = __ldg(x + r * D4 + c), v1 = __ldg(x + (r + 1) * D4 + c);
    const float m0 = __ldg(mean + r), m1 = __ldg(mean + r + 1), i0 = __ldg(invstd + r), i1 = __ldg(invstd + r + 1);
    a.x += g0.x; a.y += g0.y; a.z += g0.z; a.w += g0.w;
    a2.x += g1.x; a2.y += g1.y; a2.z += g1.z; a2.w += g1.w;
    b.x += g0.x * (v0.x - m0) * i0; b.y += g0.y * (v0.y - m0) * i0;
    b.z += g0.z * (v0.z - m0) * i0; b.w += g0.w * (v0.w - m0) * i0;
    b2.x += g1.x * (v1.x - m1) * i1; b2.y += g1.y * (v1.y - m1) * i1;
    b2.z += g1.z * (v1.z - m1) * i1; b2.w += g1.w * (v1.w - m1) * i1;
  }
  for (; r < r1; ++r) {
    const float4 g0 = __ldg(dy + r * D4 + c), v0 = __ldg(x + r * D4 + c);
    const float m0 = __ldg(mean + r), i0 = __ldg(invstd + r);
    a.x += g0.x; a.y += g0.y; a.z += g0.z; a.w += g0.w;
    b.x += g0.x * (v0.x - m0) * i0; b.y += g0.y * (v0.y - m0) * i0;
    b.z += g0.z * (v0.z - m0) * i0; b.w += g0.w * (v0.w - m0) * i0;
  }
  const long long o = (long long)ch * (D4 * 4) + 4 * c;
  *reinterpret_cast<float4*>(part + o) = make_float4(a.x + a2.x, a.y + a2.y, a.z + a2.z, a.w + a2.w);
  *reinterpret_cast<float4*>(part + PLANE_FLOATS + o) = make_float4(b.x + b2.x, b.y + b2.y, b.z + b2.z, b.w + b2.w);
}

}  // namespace

extern "C" {

int tsb_bn_forward(const float* x, const float* scale, const float* bias, float* y, float* save_mean,
                   float* save_invstd, float* run_mean, float* run_var, long long rows, long long C,
                   long long ldx, long long ldy, float momentum, float eps, int relu, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0 || C <= 0) return TSB_ERR_ARG;
  if ((C % 4) || (ldx % 4) || (ldy % 4) || C > 8192) return TSB_ERR_UNSUPPORTED;
  float* part = scratch();
  if (!part) return TSB_ERR_OOM;
  const StatGeom sg = stat_geom(rows, (int)C);
  col_partial<0><<<sg.grid, STAT_THREADS, 0, st>>>(x, nullptr, nullptr, nullptr, part, rows, (int)C, ldx, 0, sg.chunks, sg.cw);
  bn_finalize_fwd<<<fin_blocks(C), dim3(32, FIN_LANES), 0, st>>>(part, sg.chunks, (int)C, (double)rows, eps, momentum, save_mean,
                                                         save_invstd, run_mean, run_var);
  bn_apply_fwd<<<ew_grid(rows * (C / 4)), 256, 0, st>>>(x, scale, bias, save_mean, save_invstd, y, rows, (int)C,
                                                        ldx, ldy, relu);
  return done();
}

// Batch-norm forward whose column partial sums were produced by the convolution that wrote x
// (tsb_conv2d_fwd_stats): finalise + one normalise pass; x is read once instead of twice.
int tsb_bn_forward_from_partials(const float* part, int chunks, long long plane, const float* x, const float* scale,
                                 const float* bias, float* y, float* save_mean, float* save_invstd, float* run_mean,
                                 float* run_var, long long rows, long long C, long long ldx, long long ldy,
                                 float momentum, float eps, int relu, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0 || C <= 0 || chunks <= 0 || !part) return TSB_ERR_ARG;
  if ((C % 4) || (ldx % 4) || (ldy % 4)) return TSB_ERR_UNSUPPORTED;
  bn_finalize_fwd<<<fin_blocks(C), dim3(32, FIN_LANES), 0, st>>>(part, chunks, (int)C, (double)rows, eps, momentum,
                                                                 save_mean, save_invstd, run_mean, run_var, plane);
  bn_apply_fwd<<<ew_grid(rows * (C / 4)), 256, 0, st>>>(x, scale, bias, save_mean, save_invstd, y, rows, (int)C,
                                                        ldx, ldy, relu);
  return done();
}

// Normalise / scale / shift (/ReLU) with statistics that are already known: what a rematerialised
// batch-norm output needs (the statistics of the step were computed by the first forward pass, and
// the running statistics must not be updated a second time).
int tsb_bn_apply(const float* x, const float* scale, const float* bias, float* y, const float* save_mean,
                 const float* save_invstd, long long rows, long long C, long long ldx, long long ldy, int relu,
                 void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0 || C <= 0) return TSB_ERR_ARG;
  if ((C % 4) || (ldx % 4) || (ldy % 4)) return TSB_ERR_UNSUPPORTED;
  bn_apply_fwd<<<ew_grid(rows * (C / 4)), 256, 0, st>>>(x, scale, bias, save_mean, save_invstd, y, rows, (int)C,
                                                        ldx, ldy, relu);
  return done();
}

// Batch-norm forward that allocates nothing (declared and documented in norm_static.h).
int tsb_bn_forward_static(const float* x, const float* scale, const float* bias, float* y, float* save_mean,
                          float* save_invstd, float* run_mean, float* run_var, long long rows, long long C,
                          long long ldx, long long ldy, float momentum, float eps, int relu, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0 || C <= 0) return TSB_ERR_ARG;
  if (C > TSB_BN_STATIC_MAX_CHANNELS) return TSB_ERR_SCRATCH;      // partial planes would not fit
  if ((C % 4) || (ldx % 4) || (ldy % 4)) return TSB_ERR_UNSUPPORTED;
  float* part = nullptr;
  const int rc = static_scratch(&part);
  if (rc) return rc;
  const StatGeom sg = stat_geom(rows, (int)C);
  // every partial word that the finalise step reads is written by the statistics step of the
  // same call, so nothing in the shared array has to be cleared between calls
  col_partial<0><<<sg.grid, STAT_THREADS, 0, st>>>(x, nullptr, nullptr, nullptr, part, rows, (int)C, ldx, 0, sg.chunks, sg.cw);
  bn_finalize_fwd<<<fin_blocks(C), dim3(32, FIN_LANES), 0, st>>>(part, sg.chunks, (int)C, (double)rows, eps, momentum, save_mean,
                                                         save_invstd, run_mean, run_var);
  bn_apply_fwd<<<ew_grid(rows * (C / 4)), 256, 0, st>>>(x, scale, bias, save_mean, save_invstd, y, rows, (int)C,
                                                        ldx, ldy, relu);
  return done();
}

int tsb_bn_backward(const float* dy, const float* x, const float* scale, const float* save_mean,
                    const float* save_invstd, float* dx, float* dscale, float* dbias, long long rows, long long C,
                    long long ldx, long long lddy, long long lddx, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0 || C <= 0) return TSB_ERR_ARG;
  if ((C % 4) || (ldx % 4) || (lddy % 4) || (lddx % 4) || C > 8192) return TSB_ERR_UNSUPPORTED;
  float* part = scratch();
  if (!part) return TSB_ERR_OOM;
  const StatGeom sg = stat_geom(rows, (int)C);
  col_partial<1><<<sg.grid, STAT_THREADS, 0, st>>>(dy, x, save_mean, save_invstd, part, rows, (int)C, lddy, ldx, sg.chunks,
                                                   sg.cw);
  bn_finalize_bwd<<<fin_blocks(C), dim3(32, FIN_LANES), 0, st>>>(part, sg.chunks, (int)C, dscale, dbias);
  bn_apply_bwd<<<ew_grid(rows * (C / 4)), 256, 0, st>>>(dy, x, scale, save_mean, save_invstd, dscale, dbias, dx,
                                                        rows, (int)C, lddy, ldx, lddx, 1.f / (float)rows);
  return done();
}

// Backward of the fused batch-norm + ReLU.  The incoming gradient is masked on the fly in both
// passes by the sign of the forward output, which is recomputed from x, scale and bias: no separate
// ReLU-gradient pass exists and the forward output is not read at all.
int tsb_bn_relu_backward(const float* dy, const float* x, const float* scale, const float* bias,
                         const float* save_mean, const float* save_invstd, float* dx, float* dscale, float* dbias,
                         long long rows, long long C, long long ldx, long long lddy, long long lddx, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0 || C <= 0 || !bias) return TSB_ERR_ARG;
  if ((C % 4) || (ldx % 4) || (lddy % 4) || (lddx % 4) || C > 8192) return TSB_ERR_UNSUPPORTED;
  float* part = scratch();
  if (!part) return TSB_ERR_OOM;
  const StatGeom sg = stat_geom(rows, (int)C);
  col_partial<1><<<sg.grid, STAT_THREADS, 0, st>>>(dy, x, save_mean, save_invstd, part, rows, (int)C, lddy, ldx, sg.chunks,
                                                   sg.cw, scale, bias);
  bn_finalize_bwd<<<fin_blocks(C), dim3(32, FIN_LANES), 0, st>>>(part, sg.chunks, (int)C, dscale, dbias);
  bn_apply_bwd<<<ew_grid(rows * (C / 4)), 256, 0, st>>>(dy, x, scale, save_mean, save_invstd, dscale, dbias, dx,
                                                        rows, (int)C, lddy, ldx, lddx, 1.f / (float)rows, bias);
  return done();
}

// ---- batch norm over batch pieces (micro-tensors) --------------------------------------------------
// A batch norm whose input exists only one batch piece at a time takes its column sums piece by piece
// into a caller-owned partial buffer (two planes of `plane` floats; piece j fills chunk rows
// [chunk_offset, chunk_offset + *chunks_out)), finalises once over all chunk rows with the row count of
// the whole batch, and then normalises piece by piece with tsb_bn_apply.  The backward pass does the
// same with (sum dy, sum dy * xhat).  The arithmetic is the one of the whole-batch entries above: the
// partial sums are combined in double in a fixed order, so the result does not depend on the split.
int tsb_bn_stats_partial(const float* x, float* part, long long plane, int chunk_offset, int chunk_cap,
                         long long rows, long long C, long long ldx, int* chunks_out, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0 || C <= 0 || !part || !chunks_out || chunk_cap <= 0) return TSB_ERR_ARG;
  if ((C % 4) || (ldx % 4)) return TSB_ERR_UNSUPPORTED;
  const StatGeom sg = stat_geom(rows, (int)C, chunk_cap);
  if ((long long)(chunk_offset + sg.chunks) * C > plane) return TSB_ERR_SCRATCH;
  col_partial<0><<<sg.grid, STAT_THREADS, 0, st>>>(x, nullptr, nullptr, nullptr, part + (long long)chunk_offset * C,
                                                   rows, (int)C, ldx, 0, sg.chunks, sg.cw, nullptr, nullptr, plane);
  *chunks_out = sg.chunks;
  return done();
}

int tsb_bn_stats_finalize(const float* part, long long plane, int chunks, double count, long long C, float eps,
                          float momentum, float* mean, float* invstd, float* run_mean, float* run_var,
                          void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (chunks <= 0 || C <= 0 || count <= 0 || !part) return TSB_ERR_ARG;
  bn_finalize_fwd<<<fin_blocks(C), dim3(32, FIN_LANES), 0, st>>>(part, chunks, (int)C, count, eps, momentum, mean,
                                                                 invstd, run_mean, run_var, plane);
  return done();
}

// rscale / rbias non-null: the forward was the fused batch norm + ReLU (dy is masked by the sign of its output).
int tsb_bn_bwd_partial(const float* dy, const float* x, const float* mean, const float* invstd,
                       const float* rscale, const float* rbias, float* part, long long plane, int chunk_offset,
                       int chunk_cap, long long rows, long long C, long long lddy, long long ldx, int* chunks_out,
                       void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0 || C <= 0 || !part || !chunks_out || chunk_cap <= 0) return TSB_ERR_ARG;
  if ((C % 4) || (ldx % 4) || (lddy % 4)) return TSB_ERR_UNSUPPORTED;
  const StatGeom sg = stat_geom(rows, (int)C, chunk_cap);
  if ((long long)(chunk_offset + sg.chunks) * C > plane) return TSB_ERR_SCRATCH;
  col_partial<1><<<sg.grid, STAT_THREADS, 0, st>>>(dy, x, mean, invstd, part + (long long)chunk_offset * C, rows,
                                                   (int)C, lddy, ldx, sg.chunks, sg.cw, rscale, rbias, plane);
  *chunks_out = sg.chunks;
  return done();
}

int tsb_bn_bwd_finalize(const float* part, long long plane, int chunks, long long C, float* dscale, float* dbias,
                        void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (chunks <= 0 || C <= 0 || !part) return TSB_ERR_ARG;
  bn_finalize_bwd<<<fin_blocks(C), dim3(32, FIN_LANES), 0, st>>>(part, chunks, (int)C, dscale, dbias, plane);
  return done();
}

// dx of one batch piece from the whole-batch sums; total_count = rows of the WHOLE batch.
int tsb_bn_bwd_apply(const float* dy, const float* x, const float* scale, const float* rbias, const float* mean,
                     const float* invstd, const float* dscale, const float* dbias, float* dx, long long rows,
                     long long C, long long lddy, long long ldx, long long lddx, double total_count, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0 || C <= 0 || total_count <= 0) return TSB_ERR_ARG;
  if ((C % 4) || (ldx % 4) || (lddy % 4) || (lddx % 4)) return TSB_ERR_UNSUPPORTED;
  bn_apply_bwd<<<ew_grid(rows * (C / 4)), 256, 0, st>>>(dy, x, scale, mean, invstd, dscale, dbias, dx, rows, (int)C,
                                                        lddy, ldx, lddx, (float)(1.0 / total_count), rbias);
  return done();
}

int tsb_layer_norm(const float* x, const float* scale, const float* bias, float* y, float* mean, float* invstd,
                   long long rows, long long D, float eps, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0 || D <= 0) return TSB_ERR_ARG;
  const long long threads = rows * 32;
  ln_fwd<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(x, scale, bias, y, mean, invstd, rows, (int)D, eps);
  return done();
}

int tsb_layer_norm_grad(const float* dy, const float* x, const float* scale, const float* mean,
                        const float* invstd, float* dx, float* dscale, float* dbias, long long rows, long long D,
                        void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows <= 0 || D <= 0) return TSB_ERR_ARG;
  if (D > 8192) return TSB_ERR_UNSUPPORTED;
  float* part = scratch();
  if (!part) return TSB_ERR_OOM;
  const long long threads = rows * 32;
  ln_bwd_dx<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(dy, x, scale, mean, invstd, dx, rows, (int)D);
  int chunks = (int)((rows + 31) / 32);
  if (chunks > MAX_CHUNKS) chunks = MAX_CHUNKS;
  if ((D & 3) == 0 && ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
    const int D4 = (int)(D / 4);
    const int bt = D4 >= 128 ? 128 : (D4 >= 64 ? 64 : 32);
    // about 16 rows per thread; a plane of partials holds PLANE_FLOATS / D chunks
    long long c4 = (rows + 15) / 16;
    if (c4 > PLANE_FLOATS / D) c4 = PLANE_FLOATS / D;
    if (c4 > 1024) c4 = 1024;
    chunks = (int)(c4 < 1 ? 1 : c4);
    dim3 grid4((unsigned)((D4 + bt - 1) / bt), chunks);
    ln_bwd_params_partial_v4<<<grid4, bt, 0, st>>>(reinterpret_cast<const float4*>(dy),
                                                   reinterpret_cast<const float4*>(x), mean, invstd, part, rows, D4,
                                                   chunks);
    bn_finalize_bwd<<<fin_blocks(D), dim3(32, FIN_LANES), 0, st>>>(part, chunks, (int)D, dscale, dbias);
    return done();
  }
  dim3 grid((unsigned)((D + 127) / 128), chunks);
  ln_bwd_params_partial<<<grid, 128, 0, st>>>(dy, x, mean, invstd, part, rows, (int)D, chunks);
  bn_finalize_bwd<<<fin_blocks(D), dim3(32, FIN_LANES), 0, st>>>(part, chunks, (int)D, dscale, dbias);
  return done();
}

}  // extern "C"
