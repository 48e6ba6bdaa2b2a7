// Pooling (channels-last), softmax, softmax cross-entropy (+ gradient).
//
// Pooling: one thread per (pixel, 4-channel vector), 16-byte accesses.  The max
// gradient is a gather over the windows containing an input pixel and gives the
// gradient to the FIRST maximum of each window (row-major), so it is
// deterministic, needs no atomics and no zero-fill pass.
// Softmax family: one warp per row for short rows (the row stays in registers), one
// CTA per row with 16-byte lanes and a one-pass running (max, sum) for long rows; the
// mean of the row losses is a fixed-order second stage.
//
// Roles in the reference: cudnnPoolingForward/Backward (src/ops/CudnnMaxPool.cu,
// CudnnAvgPool.cu) and the <<<1,1024>>> kernels of src/ops/Softmax.cu:3-22 and
// src/ops/SoftmaxCrossEntropy.cu:5-104.
#include <cuda_runtime.h>
#include "scratch.h"
#include <float.h>
#include <stdint.h>

#define TSB_OK 0
#define TSB_ERR_ARG 1
#define TSB_ERR_UNSUPPORTED 2
#define TSB_ERR_LAUNCH 3
#define TSB_ERR_OOM 5

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

struct PoolP {
  int n, c, h, w, oh, ow, kh, kw, pad, stride;
  long long xsn, xsh, xsw, ysn, ysh, ysw;
};

template <int KIND>
__global__ void pool_fwd(const float* __restrict__ x, float* __restrict__ y, const PoolP p) {
  const int C4 = p.c >> 2;
  const long long total = (long long)p.n * p.oh * p.ow * C4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C4) * 4;
    long long r = i / C4;
    const int ox = (int)(r % p.ow); r /= p.ow;
    const int oy = (int)(r % p.oh);
    const int n = (int)(r / p.oh);
    float4 acc = KIND == 0 ? make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX) : make_float4(0, 0, 0, 0);
    for (int a = 0; a < p.kh; ++a) {
      const int iy = oy * p.stride - p.pad + a;
      if ((unsigned)iy >= (unsigned)p.h) continue;
      for (int b = 0; b < p.kw; ++b) {
        const int ix = ox * p.stride - p.pad + b;
        if ((unsigned)ix >= (unsigned)p.w) continue;
        const float4 v = *reinterpret_cast<const float4*>(x + n * p.xsn + iy * p.xsh + ix * p.xsw + c);
        if (KIND == 0) {
          acc.x = fmaxf(acc.x, v.x); acc.y = fmaxf(acc.y, v.y); acc.z = fmaxf(acc.z, v.z); acc.w = fmaxf(acc.w, v.w);
        } else {
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
      }
    }
    if (KIND == 1) {
      const float s = 1.f / (float)(p.kh * p.kw);
      acc.x *= s; acc.y *= s; acc.z *= s; acc.w *= s;
    }
    *reinterpret_cast<float4*>(y + n * p.ysn + oy * p.ysh + ox * p.ysw + c) = acc;
  }
}

__device__ __forceinline__ int ceil_div_pos(int a, int b) { return a <= 0 ? 0 : (a + b - 1) / b; }

template <int KIND>
__global__ void pool_bwd(const float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ dy,
                         float* __restrict__ dx, const PoolP p) {
  const int C4 = p.c >> 2;
  const long long total = (long long)p.n * p.h * p.w * C4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C4) * 4;
    long long r = i / C4;
    const int ix = (int)(r % p.w); r /= p.w;
    const int iy = (int)(r % p.h);
    const int n = (int)(r / p.h);
    // output windows that contain (iy, ix)
    const int oy0 = ceil_div_pos(iy + p.pad - p.kh + 1, p.stride), oy1 = min(p.oh - 1, (iy + p.pad) / p.stride);
    const int ox0 = ceil_div_pos(ix + p.pad - p.kw + 1, p.stride), ox1 = min(p.ow - 1, (ix + p.pad) / p.stride);
    float4 acc = make_float4(0, 0, 0, 0);
    float4 me = make_float4(0, 0, 0, 0);
    if (KIND == 0) me = *reinterpret_cast<const float4*>(x + n * p.xsn + iy * p.xsh + ix * p.xsw + c);
    for (int oy = oy0; oy <= oy1; ++oy) {
      for (int ox = ox0; ox <= ox1; ++ox) {
        const float4 g = *reinterpret_cast<const float4*>(dy + n * p.ysn + oy * p.ysh + ox * p.ysw + c);
        if (KIND == 1) {
          acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
          continue;
        }
        const float4 m = *reinterpret_cast<const float4*>(y + n * p.ysn + oy * p.ysh + ox * p.ysw + c);
        // am I the first maximum of this window?  (scan the elements that precede me)
        bool fx = me.x == m.x, fy = me.y == m.y, fz = me.z == m.z, fw = me.w == m.w;
        if (fx | fy | fz | fw) {
          const int my_a = iy - (oy * p.stride - p.pad), my_b = ix - (ox * p.stride - p.pad);
          for (int a = 0; a <= my_a; ++a) {
            const int yy = oy * p.stride - p.pad + a;
            if ((unsigned)yy >= (unsigned)p.h) continue;
            const int bend = (a == my_a) ? my_b : p.kw;
            for (int b = 0; b < bend; ++b) {
              const int xx = ox * p.stride - p.pad + b;
              if ((unsigned)xx >= (unsigned)p.w) continue;
              const float4 v = *reinterpret_cast<const float4*>(x + n * p.xsn + yy * p.xsh + xx * p.xsw + c);
              fx = fx && v.x != m.x; fy = fy && v.y != m.y; fz = fz && v.z != m.z; fw = fw && v.w != m.w;
            }
          }
          if (fx) acc.x += g.x;
          if (fy) acc.y += g.y;
          if (fz) acc.z += g.z;
          if (fw) acc.w += g.w;
        }
      }
    }
    if (KIND == 1) {
      const float s = 1.f / (float)(p.kh * p.kw);
      acc.x *= s; acc.y *= s; acc.z *= s; acc.w *= s;
    }
    *reinterpret_cast<float4*>(dx + n * p.xsn + iy * p.xsh + ix * p.xsw + c) = acc;
  }
}

// Backward for windows that tile the input exactly (kernel == stride, no padding, h = oh*stride):
// one thread owns one output window and four channels, reads its K x K inputs and one gradient,
// and writes the K x K input gradients -- x and dx cross HBM once each and y is not read at all.
// Ties go to the first maximum in scan order, as in the general kernel.
template <int KIND, int K>
__global__ void pool_bwd_tiled(const float* __restrict__ x, const float* __restrict__ dy, float* __restrict__ dx,
                               const PoolP p) {
  const int C4 = p.c >> 2;
  const long long total = (long long)p.n * p.oh * p.ow * C4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C4) * 4;
    long long r = i / C4;
    const int ox = (int)(r % p.ow); r /= p.ow;
    const int oy = (int)(r % p.oh);
    const int n = (int)(r / p.oh);
    const float4 g = *reinterpret_cast<const float4*>(dy + n * p.ysn + oy * p.ysh + ox * p.ysw + c);
    const long long base = n * p.xsn + (long long)(oy * K) * p.xsh + (long long)(ox * K) * p.xsw + c;
    if (KIND == 1) {
      const float s = 1.f / (float)(K * K);
      const float4 o = make_float4(g.x * s, g.y * s, g.z * s, g.w * s);
#pragma unroll
      for (int a = 0; a < K; ++a)
#pragma unroll
        for (int b = 0; b < K; ++b) *reinterpret_cast<float4*>(dx + base + a * p.xsh + b * p.xsw) = o;
      continue;
    }
    float4 v[K * K];
#pragma unroll
    for (int a = 0; a < K; ++a)
#pragma unroll
      for (int b = 0; b < K; ++b) v[a * K + b] = *reinterpret_cast<const float4*>(x + base + a * p.xsh + b * p.xsw);
    int ax = 0, ay = 0, az = 0, aw = 0;          // index of the first maximum per channel
    float4 m = v[0];
#pragma unroll
    for (int q = 1; q < K * K; ++q) {
      if (v[q].x > m.x) { m.x = v[q].x; ax = q; }
      if (v[q].y > m.y) { m.y = v[q].y; ay = q; }
      if (v[q].z > m.z) { m.z = v[q].z; az = q; }
      if (v[q].w > m.w) { m.w = v[q].w; aw = q; }
    }
#pragma unroll
    for (int a = 0; a < K; ++a)
#pragma unroll
      for (int b = 0; b < K; ++b) {
        const int q = a * K + b;
        const float4 o = make_float4(ax == q ? g.x : 0.f, ay == q ? g.y : 0.f, az == q ? g.z : 0.f,
                                     aw == q ? g.w : 0.f);
        *reinterpret_cast<float4*>(dx + base + a * p.xsh + b * p.xsw) = o;
      }
  }
}

// Max-pool backward for windows that overlap (e.g. 3x3 stride 2), in two passes without scans:
//   pass 1, one thread per output window and four channels: position (a * kw + b) of the first
//           maximum inside the window, one byte per channel;
//   pass 2, one thread per input pixel and four channels: add dy of every window that contains the
//           pixel and whose recorded position is this pixel, in a fixed order.
// After a ReLU most windows tie at zero, which made the scan-for-earlier-maximum form of the general
// kernel expensive; here every tensor is read once.
__global__ void pool_argmax(const float* __restrict__ x, unsigned char* __restrict__ idx, const PoolP p) {
  const int C4 = p.c >> 2;
  const long long total = (long long)p.n * p.oh * p.ow * C4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C4) * 4;
    long long r = i / C4;
    const int ox = (int)(r % p.ow); r /= p.ow;
    const int oy = (int)(r % p.oh);
    const int n = (int)(r / p.oh);
    float4 m = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
    uchar4 q = make_uchar4(255, 255, 255, 255);
    for (int a = 0; a < p.kh; ++a) {
      const int iy = oy * p.stride - p.pad + a;
      if ((unsigned)iy >= (unsigned)p.h) continue;
      for (int b = 0; b < p.kw; ++b) {
        const int ix = ox * p.stride - p.pad + b;
        if ((unsigned)ix >= (unsigned)p.w) continue;
        const float4 v = *reinterpret_cast<const float4*>(x + n * p.xsn + iy * p.xsh + ix * p.xsw + c);
        const unsigned char pos = (unsigned char)(a * p.kw + b);
        if (v.x > m.x || q.x == 255) { m.x = v.x; q.x = pos; }
        if (v.y > m.y || q.y == 255) { m.y = v.y; q.y = pos; }
        if (v.z > m.z || q.z == 255) { m.z = v.z; q.z = pos; }
        if (v.w > m.w || q.w == 255) { m.w = v.w; q.w = pos; }
      }
    }
    *reinterpret_cast<uchar4*>(idx + i * 4) = q;
  }
}

__global__ void pool_bwd_from_argmax(const unsigned char* __restrict__ idx, const float* __restrict__ dy,
                                     float* __restrict__ dx, const PoolP p) {
  const int C4 = p.c >> 2;
  const long long total = (long long)p.n * p.h * p.w * C4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c4 = (int)(i % C4);
    const int c = c4 * 4;
    long long r = i / C4;
    const int ix = (int)(r % p.w); r /= p.w;
    const int iy = (int)(r % p.h);
    const int n = (int)(r / p.h);
    const int oy0 = ceil_div_pos(iy + p.pad - p.kh + 1, p.stride), oy1 = min(p.oh - 1, (iy + p.pad) / p.stride);
    const int ox0 = ceil_div_pos(ix + p.pad - p.kw + 1, p.stride), ox1 = min(p.ow - 1, (ix + p.pad) / p.stride);
    float4 acc = make_float4(0, 0, 0, 0);
    for (int oy = oy0; oy <= oy1; ++oy) {
      for (int ox = ox0; ox <= ox1; ++ox) {
        const int pos = (iy - (oy * p.stride - p.pad)) * p.kw + (ix - (ox * p.stride - p.pad));
        const uchar4 q = *reinterpret_cast<const uchar4*>(idx + ((((long long)n * p.oh + oy) * p.ow + ox) * C4 + c4) * 4);
        const float4 g = *reinterpret_cast<const float4*>(dy + n * p.ysn + oy * p.ysh + ox * p.ysw + c);
        if (q.x == pos) acc.x += g.x;
        if (q.y == pos) acc.y += g.y;
        if (q.z == pos) acc.z += g.z;
        if (q.w == pos) acc.w += g.w;
      }
    }
    *reinterpret_cast<float4*>(dx + n * p.xsn + iy * p.xsh + ix * p.xsw + c) = acc;
  }
}

unsigned char* argmax_scratch(size_t bytes) {
  return static_cast<unsigned char*>(tsb_scratch::get(nullptr, tsb_scratch::POOL_ARGMAX, bytes, size_t(32) << 20));
}

// ------------------------------------------------------------------ softmax family
__device__ __forceinline__ float block_max(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = sh[0];
  for (int i = 1; i < (blockDim.x >> 5); ++i) r = fmaxf(r, sh[i]);
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) r += sh[i];
  __syncthreads();
  return r;
}

__global__ void softmax_rows(const float* __restrict__ x, float* __restrict__ y, long long rows, long long cols) {
  __shared__ float sh[8];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    float m = -FLT_MAX;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) m = fmaxf(m, xr[i]);
    m = block_max(m, sh);
    float s = 0.f;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) s += __expf(xr[i] - m);
    s = block_sum(s, sh);
    const float inv = 1.f / s;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) y[row * cols + i] = __expf(xr[i] - m) * inv;
  }
}

// Short rows (cols <= 1024, a multiple of 4): one warp per row, the row held in registers between the
// maximum, the sum and the store, so it is read once and no block barrier is involved.
template <int NV>
__global__ void __launch_bounds__(256) softmax_warp_rows(const float4* __restrict__ x, float4* __restrict__ y,
                                                         long long rows, int nvec) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarp = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarp) {
    const float4* xr = x + row * nvec;
    float4 v[NV];
    float m = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + 32 * j;
      v[j] = i < nvec ? __ldg(xr + i) : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
      m = fmaxf(m, fmaxf(fmaxf(v[j].x, v[j].y), fmaxf(v[j].z, v[j].w)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      v[j].x = __expf(v[j].x - m); v[j].y = __expf(v[j].y - m);
      v[j].z = __expf(v[j].z - m); v[j].w = __expf(v[j].w - m);
      s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float inv = 1.f / s;
    float4* yr = y + row * nvec;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + 32 * j;
      if (i < nvec) yr[i] = make_float4(v[j].x * inv, v[j].y * inv, v[j].z * inv, v[j].w * inv);
    }
  }
}

// The same for rows whose length is no multiple of 4 (or whose base is not 16-byte aligned): scalar,
// still coalesced, lanes; NE elements per lane.
template <int NE>
__global__ void __launch_bounds__(256) softmax_warp_rows_scalar(const float* __restrict__ x, float* __restrict__ y,
                                                                long long rows, int cols) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarp = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarp) {
    const float* xr = x + row * cols;
    float v[NE];
    float m = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < NE; ++j) {
      const int i = lane + 32 * j;
      v[j] = i < cols ? __ldg(xr + i) : -FLT_MAX;
      m = fmaxf(m, v[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NE; ++j) { v[j] = __expf(v[j] - m); s += v[j]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float inv = 1.f / s;
    float* yr = y + row * cols;
#pragma unroll
    for (int j = 0; j < NE; ++j) {
      const int i = lane + 32 * j;
      if (i < cols) yr[i] = v[j] * inv;
    }
  }
}

template <int NE>
__global__ void __launch_bounds__(256) softmax_grad_warp_rows_scalar(const float* __restrict__ y,
                                                                     const float* __restrict__ dy,
                                                                     float* __restrict__ dx, long long rows,
                                                                     int cols) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarp = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarp) {
    const float* yr = y + row * cols;
    const float* gr = dy + row * cols;
    float a[NE], g[NE];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NE; ++j) {
      const int i = lane + 32 * j;
      a[j] = i < cols ? __ldg(yr + i) : 0.f;
      g[j] = i < cols ? __ldg(gr + i) : 0.f;
      s += a[j] * g[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    float* dr = dx + row * cols;
#pragma unroll
    for (int j = 0; j < NE; ++j) {
      const int i = lane + 32 * j;
      if (i < cols) dr[i] = a[j] * (g[j] - s);
    }
  }
}

// Softmax backward, dx = y * (dy - sum(dy * y)): one warp per row, y and dy read once.
template <int NV>
__global__ void __launch_bounds__(256) softmax_grad_warp_rows(const float4* __restrict__ y,
                                                              const float4* __restrict__ dy,
                                                              float4* __restrict__ dx, long long rows, int nvec) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarp = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarp) {
    const float4* yr = y + row * nvec;
    const float4* gr = dy + row * nvec;
    float4 a[NV], g[NV];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + 32 * j;
      a[j] = i < nvec ? __ldg(yr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      g[j] = i < nvec ? __ldg(gr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      s += (a[j].x * g[j].x + a[j].y * g[j].y) + (a[j].z * g[j].z + a[j].w * g[j].w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    float4* dr = dx + row * nvec;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + 32 * j;
      if (i < nvec)
        dr[i] = make_float4(a[j].x * (g[j].x - s), a[j].y * (g[j].y - s), a[j].z * (g[j].z - s),
                            a[j].w * (g[j].w - s));
    }
  }
}

// Attention soft-max: y = softmax(scale * x + mask) over rows of `cols` scores, one warp per row, the row held in
// registers, so the scaling, the key-padding mask and the causal mask cost no pass of their own.
//   key_tokens (optional) [batch][cols]: a key whose token is 0 is padding and gets -1e9 added
//   causal: column j of query row q (row % tq) is replaced by -1e9 when j > q
// Rows are [batch][rows_per_batch] with rows_per_batch = heads * tq.
template <int NE>
__global__ void __launch_bounds__(256) masked_softmax_warp_rows(const float* __restrict__ x,
                                                                const float* __restrict__ key_tokens,
                                                                float* __restrict__ y, long long rows, int cols,
                                                                long long rows_per_batch, int tq, float scale,
                                                                int causal) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarp = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarp) {
    const float* xr = x + row * cols;
    // 32-bit index arithmetic (rows < 2^31, checked by the launcher): two 64-bit divisions per row would cost as much
    // as the row's loads
    const float* kt = key_tokens ? key_tokens + (long long)((unsigned)row / (unsigned)rows_per_batch) * cols : nullptr;
    const int q = (int)((unsigned)row % (unsigned)tq);
    float v[NE];
    float m = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < NE; ++j) {
      const int i = lane + 32 * j;
      float t = -FLT_MAX;
      if (i < cols) {
        t = __ldg(xr + i) * scale;
        if (kt && __ldg(kt + i) == 0.f) t += -1e9f;
        if (causal && i > q) t = -1e9f;
      }
      v[j] = t;
      m = fmaxf(m, t);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NE; ++j) {
      const int i = lane + 32 * j;
      v[j] = i < cols ? __expf(v[j] - m) : 0.f;
      s += v[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float inv = 1.f / s;
    float* yr = y + row * cols;
#pragma unroll
    for (int j = 0; j < NE; ++j) {
      const int i = lane + 32 * j;
      if (i < cols) yr[i] = v[j] * inv;
    }
  }
}

// The same with 16-byte lanes (cols % 4 == 0, 16-byte aligned rows): NV float4 per lane.
template <int NV>
__global__ void __launch_bounds__(256) masked_softmax_warp_rows_v4(const float4* __restrict__ x,
                                                                   const float4* __restrict__ key_tokens,
                                                                   float4* __restrict__ y, long long rows, int nvec,
                                                                   long long rows_per_batch, int tq, float scale,
                                                                   int causal) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarp = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarp) {
    const float4* xr = x + row * nvec;
    const float4* kt = key_tokens ? key_tokens + (long long)((unsigned)row / (unsigned)rows_per_batch) * nvec : nullptr;
    const int q = (int)((unsigned)row % (unsigned)tq);
    float4 v[NV];
    float m = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + 32 * j;
      float4 t = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
      if (i < nvec) {
        t = __ldg(xr + i);
        t.x *= scale; t.y *= scale; t.z *= scale; t.w *= scale;
        if (kt) {
          const float4 k = __ldg(kt + i);
          if (k.x == 0.f) t.x += -1e9f;
          if (k.y == 0.f) t.y += -1e9f;
          if (k.z == 0.f) t.z += -1e9f;
          if (k.w == 0.f) t.w += -1e9f;
        }
        if (causal) {
          const int c = 4 * i;
          if (c > q) t.x = -1e9f;
          if (c + 1 > q) t.y = -1e9f;
          if (c + 2 > q) t.z = -1e9f;
          if (c + 3 > q) t.w = -1e9f;
        }
      }
      v[j] = t;
      m = fmaxf(m, fmaxf(fmaxf(t.x, t.y), fmaxf(t.z, t.w)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + 32 * j;
      if (i < nvec) {
        v[j].x = __expf(v[j].x - m); v[j].y = __expf(v[j].y - m);
        v[j].z = __expf(v[j].z - m); v[j].w = __expf(v[j].w - m);
      } else {
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float inv = 1.f / s;
    float4* yr = y + row * nvec;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + 32 * j;
      if (i < nvec) yr[i] = make_float4(v[j].x * inv, v[j].y * inv, v[j].z * inv, v[j].w * inv);
    }
  }
}

// Its backward: dx = scale * y * (dy - sum(dy * y)) (masked positions have y = 0).
template <int NE>
__global__ void __launch_bounds__(256) scaled_softmax_grad_warp_rows(const float* __restrict__ y,
                                                                     const float* __restrict__ dy,
                                                                     float* __restrict__ dx, long long rows, int cols,
                                                                     float scale) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarp = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarp) {
    const float* yr = y + row * cols;
    const float* gr = dy + row * cols;
    float a[NE], g[NE];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NE; ++j) {
      const int i = lane + 32 * j;
      a[j] = i < cols ? __ldg(yr + i) : 0.f;
      g[j] = i < cols ? __ldg(gr + i) : 0.f;
      s += a[j] * g[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    float* dr = dx + row * cols;
#pragma unroll
    for (int j = 0; j < NE; ++j) {
      const int i = lane + 32 * j;
      if (i < cols) dr[i] = scale * a[j] * (g[j] - s);
    }
  }
}

template <int NV>
__global__ void __launch_bounds__(256) scaled_softmax_grad_warp_rows_v4(const float4* __restrict__ y,
                                                                        const float4* __restrict__ dy,
                                                                        float4* __restrict__ dx, long long rows,
                                                                        int nvec, float scale) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarp = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarp) {
    const float4* yr = y + row * nvec;
    const float4* gr = dy + row * nvec;
    float4 a[NV], g[NV];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + 32 * j;
      a[j] = i < nvec ? __ldg(yr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      g[j] = i < nvec ? __ldg(gr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      s += (a[j].x * g[j].x + a[j].y * g[j].y) + (a[j].z * g[j].z + a[j].w * g[j].w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    float4* dr = dx + row * nvec;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + 32 * j;
      if (i < nvec)
        dr[i] = make_float4(scale * a[j].x * (g[j].x - s), scale * a[j].y * (g[j].y - s),
                            scale * a[j].z * (g[j].z - s), scale * a[j].w * (g[j].w - s));
    }
  }
}

// Any row length: one CTA per row, the second pass finds the row in L2.
__global__ void softmax_grad_rows(const float* __restrict__ y, const float* __restrict__ dy, float* __restrict__ dx,
                                  long long rows, long long cols) {
  __shared__ float sh[8];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* yr = y + row * cols;
    const float* gr = dy + row * cols;
    float s = 0.f;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) s += yr[i] * gr[i];
    s = block_sum(s, sh);
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) dx[row * cols + i] = yr[i] * (gr[i] - s);
  }
}

// Running (maximum, sum of exponentials) of a row in one pass: the sum is rescaled when the maximum moves.
struct MaxSum { float m, s; };
__device__ __forceinline__ MaxSum ms_join(MaxSum a, MaxSum b) {
  const float m = fmaxf(a.m, b.m);
  return {m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}
__device__ __forceinline__ void ms_add4(MaxSum& a, const float4 v) {
  const float m4 = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
  if (m4 > a.m) { a.s *= __expf(a.m - m4); a.m = m4; }
  a.s += (__expf(v.x - a.m) + __expf(v.y - a.m)) + (__expf(v.z - a.m) + __expf(v.w - a.m));
}
// Block-wide join; sh holds 2 floats per warp.
__device__ __forceinline__ MaxSum block_max_sum(MaxSum a, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum b{__shfl_xor_sync(0xffffffffu, a.m, o), __shfl_xor_sync(0xffffffffu, a.s, o)};
    a = ms_join(a, b);
  }
  if (lane == 0) { sh[2 * w] = a.m; sh[2 * w + 1] = a.s; }
  __syncthreads();
  MaxSum r{sh[0], sh[1]};
  for (int i = 1; i < nw; ++i) r = ms_join(r, MaxSum{sh[2 * i], sh[2 * i + 1]});
  __syncthreads();
  return r;
}
__device__ __forceinline__ MaxSum row_max_sum(const float4* __restrict__ xr, int nvec, float* sh) {
  MaxSum a{-FLT_MAX, 0.f};
  int i = threadIdx.x;
  for (; i + 3 * (int)blockDim.x < nvec; i += 4 * blockDim.x) {
    const float4 v0 = __ldg(xr + i), v1 = __ldg(xr + i + blockDim.x), v2 = __ldg(xr + i + 2 * blockDim.x),
                 v3 = __ldg(xr + i + 3 * blockDim.x);
    ms_add4(a, v0); ms_add4(a, v1); ms_add4(a, v2); ms_add4(a, v3);
  }
  for (; i < nvec; i += blockDim.x) ms_add4(a, __ldg(xr + i));
  return block_max_sum(a, sh);
}

// Long rows, 16-byte lanes: the logits come from DRAM once (the second pass finds the row in L2, the
// rows in flight being kept below its size by the block size chosen at launch).
__global__ void __launch_bounds__(512) ce_rows_v4(const float4* __restrict__ x, const float4* __restrict__ lab,
                                                  float* __restrict__ row_loss, long long rows, int nvec) {
  __shared__ float sh[64];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float4* xr = x + row * nvec;
    const float4* lr = lab + row * nvec;
    const MaxSum ms = row_max_sum(xr, nvec, sh);
    const float lse = ms.m + logf(ms.s);
    float l = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const float4 t = __ldcs(lr + i);
      const float4 v = __ldg(xr + i);
      l -= (t.x * (v.x - lse) + t.y * (v.y - lse)) + (t.z * (v.z - lse) + t.w * (v.w - lse));
    }
    l = block_sum(l, sh);
    if (threadIdx.x == 0) row_loss[row] = l;
  }
}

__global__ void __launch_bounds__(512) ce_grad_rows_v4(const float4* __restrict__ x, const float4* __restrict__ lab,
                                                       const float* __restrict__ g, float4* __restrict__ dx,
                                                       long long rows, int nvec) {
  __shared__ float sh[64];
  const float scale = g[0] / (float)rows;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float4* xr = x + row * nvec;
    const float4* lr = lab + row * nvec;
    float4* dr = dx + row * nvec;
    const MaxSum ms = row_max_sum(xr, nvec, sh);
    const float inv = 1.f / ms.s, m = ms.m;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const float4 t = __ldcs(lr + i);
      const float4 v = __ldg(xr + i);
      float4 o;
      o.x = (__expf(v.x - m) * inv - t.x) * scale;
      o.y = (__expf(v.y - m) * inv - t.y) * scale;
      o.z = (__expf(v.z - m) * inv - t.z) * scale;
      o.w = (__expf(v.w - m) * inv - t.w) * scale;
      __stcs(dr + i, o);
    }
  }
}

__global__ void ce_rows(const float* __restrict__ x, const float* __restrict__ lab, float* __restrict__ row_loss,
                        long long rows, long long cols) {
  __shared__ float sh[8];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    const float* lr = lab + row * cols;
    float m = -FLT_MAX;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) m = fmaxf(m, xr[i]);
    m = block_max(m, sh);
    float s = 0.f;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) s += expf(xr[i] - m);
    s = block_sum(s, sh);
    const float lse = m + logf(s);
    float l = 0.f;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) l -= lr[i] * (xr[i] - lse);
    l = block_sum(l, sh);
    if (threadIdx.x == 0) row_loss[row] = l;
  }
}

__global__ void mean_rows(const float* __restrict__ row_loss, float* __restrict__ out, long long rows) {
  __shared__ float sh[32];
  float s = 0.f;
  for (long long i = threadIdx.x; i < rows; i += blockDim.x) s += row_loss[i];
  s = block_sum(s, sh);
  if (threadIdx.x == 0) out[0] = s / (float)rows;
}

__global__ void ce_grad_rows(const float* __restrict__ x, const float* __restrict__ lab, const float* __restrict__ g,
                             float* __restrict__ dx, long long rows, long long cols) {
  __shared__ float sh[8];
  const float scale = g[0] / (float)rows;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    float m = -FLT_MAX;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) m = fmaxf(m, xr[i]);
    m = block_max(m, sh);
    float s = 0.f;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) s += expf(xr[i] - m);
    s = block_sum(s, sh);
    const float inv = 1.f / s;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x)
      dx[row * cols + i] = (expf(xr[i] - m) * inv - lab[row * cols + i]) * scale;
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

float* row_scratch(long long rows) {
  return static_cast<float*>(tsb_scratch::get(nullptr, tsb_scratch::LOSS_ROWS, (size_t)rows * sizeof(float),
                                              size_t(65536) * sizeof(float)));
}

}  // namespace

extern "C" {

int tsb_pool_fwd(int kind, const float* x, float* y, int n, int c, int h, int w, int oh, int ow, int kh, int kw,
                 int pad, int stride, long long xsn, long long xsh, long long xsw, long long ysn, long long ysh,
                 long long ysw, void* stream) {
  if ((c % 4) || (xsw % 4) || (ysw % 4)) return TSB_ERR_UNSUPPORTED;
  PoolP p{n, c, h, w, oh, ow, kh, kw, pad, stride, xsn, xsh, xsw, ysn, ysh, ysw};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = ew_grid((long long)n * oh * ow * (c / 4));
  if (kind == 0) pool_fwd<0><<<grid, 256, 0, st>>>(x, y, p);
  else pool_fwd<1><<<grid, 256, 0, st>>>(x, y, p);
  return done();
}

int tsb_pool_bwd(int kind, const float* x, const float* y, const float* dy, float* dx, int n, int c, int h, int w,
                 int oh, int ow, int kh, int kw, int pad, int stride, long long xsn, long long xsh, long long xsw,
                 long long ysn, long long ysh, long long ysw, void* stream) {
  if ((c % 4) || (xsw % 4) || (ysw % 4)) return TSB_ERR_UNSUPPORTED;
  if (kind == 0 && (!x || !y)) return TSB_ERR_ARG;
  PoolP p{n, c, h, w, oh, ow, kh, kw, pad, stride, xsn, xsh, xsw, ysn, ysh, ysw};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (kh == stride && kw == stride && pad == 0 && oh * stride == h && ow * stride == w && (stride == 2 || stride == 3)) {
    const int tg = ew_grid((long long)n * oh * ow * (c / 4));
    if (kind == 0 && stride == 2) pool_bwd_tiled<0, 2><<<tg, 256, 0, st>>>(x, dy, dx, p);
    else if (kind == 0) pool_bwd_tiled<0, 3><<<tg, 256, 0, st>>>(x, dy, dx, p);
    else if (stride == 2) pool_bwd_tiled<1, 2><<<tg, 256, 0, st>>>(x, dy, dx, p);
    else pool_bwd_tiled<1, 3><<<tg, 256, 0, st>>>(x, dy, dx, p);
    return done();
  }
  const int grid = ew_grid((long long)n * h * w * (c / 4));
  if (kind == 0 && kh * kw < 255) {
    // overlapping windows: positions of the maxima first, then a gather per input pixel (one scratch
    // buffer per device: pooling backward passes of one device must not overlap on different streams)
    unsigned char* idx = argmax_scratch((size_t)n * oh * ow * c);
    if (idx) {
      pool_argmax<<<ew_grid((long long)n * oh * ow * (c / 4)), 256, 0, st>>>(x, idx, p);
      pool_bwd_from_argmax<<<grid, 256, 0, st>>>(idx, dy, dx, p);
      return done();
    }
  }
  if (kind == 0) pool_bwd<0><<<grid, 256, 0, st>>>(x, y, dy, dx, p);
  else pool_bwd<1><<<grid, 256, 0, st>>>(x, y, dy, dx, p);
  return done();
}

int tsb_softmax(const float* x, float* y, long long rows, long long cols, void* stream) {
  if (rows <= 0 || cols <= 0) return TSB_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cols <= 1024 && cols % 4 == 0 && aligned16(x) && aligned16(y)) {
    const int nvec = (int)(cols / 4);
    const long long blocks = (rows + 7) / 8;
    const int wgrid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
    const float4* xv = reinterpret_cast<const float4*>(x);
    float4* yv = reinterpret_cast<float4*>(y);
    if (nvec <= 32) softmax_warp_rows<1><<<wgrid, 256, 0, st>>>(xv, yv, rows, nvec);
    else if (nvec <= 64) softmax_warp_rows<2><<<wgrid, 256, 0, st>>>(xv, yv, rows, nvec);
    else if (nvec <= 128) softmax_warp_rows<4><<<wgrid, 256, 0, st>>>(xv, yv, rows, nvec);
    else softmax_warp_rows<8><<<wgrid, 256, 0, st>>>(xv, yv, rows, nvec);
    return done();
  }
  if (cols <= 1024) {
    const long long blocks = (rows + 7) / 8;
    const int wgrid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
    const int c = (int)cols;
    if (c <= 64) softmax_warp_rows_scalar<2><<<wgrid, 256, 0, st>>>(x, y, rows, c);
    else if (c <= 128) softmax_warp_rows_scalar<4><<<wgrid, 256, 0, st>>>(x, y, rows, c);
    else if (c <= 256) softmax_warp_rows_scalar<8><<<wgrid, 256, 0, st>>>(x, y, rows, c);
    else if (c <= 512) softmax_warp_rows_scalar<16><<<wgrid, 256, 0, st>>>(x, y, rows, c);
    else softmax_warp_rows_scalar<32><<<wgrid, 256, 0, st>>>(x, y, rows, c);
    return done();
  }
  const int grid = (int)(rows < 148 * 16 ? rows : 148 * 16);
  softmax_rows<<<grid, cols >= 1024 ? 256 : 128, 0, st>>>(x, y, rows, cols);
  return done();
}

int tsb_softmax_grad(const float* y, const float* dy, float* dx, long long rows, long long cols, void* stream) {
  if (rows <= 0 || cols <= 0) return TSB_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cols <= 1024 && cols % 4 == 0 && aligned16(y) && aligned16(dy) && aligned16(dx)) {
    const int nvec = (int)(cols / 4);
    const long long blocks = (rows + 7) / 8;
    const int wgrid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
    const float4* yv = reinterpret_cast<const float4*>(y);
    const float4* gv = reinterpret_cast<const float4*>(dy);
    float4* dv = reinterpret_cast<float4*>(dx);
    if (nvec <= 32) softmax_grad_warp_rows<1><<<wgrid, 256, 0, st>>>(yv, gv, dv, rows, nvec);
    else if (nvec <= 64) softmax_grad_warp_rows<2><<<wgrid, 256, 0, st>>>(yv, gv, dv, rows, nvec);
    else if (nvec <= 128) softmax_grad_warp_rows<4><<<wgrid, 256, 0, st>>>(yv, gv, dv, rows, nvec);
    else softmax_grad_warp_rows<8><<<wgrid, 256, 0, st>>>(yv, gv, dv, rows, nvec);
    return done();
  }
  if (cols <= 1024) {
    const long long blocks = (rows + 7) / 8;
    const int wgrid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
    const int c = (int)cols;
    if (c <= 64) softmax_grad_warp_rows_scalar<2><<<wgrid, 256, 0, st>>>(y, dy, dx, rows, c);
    else if (c <= 128) softmax_grad_warp_rows_scalar<4><<<wgrid, 256, 0, st>>>(y, dy, dx, rows, c);
    else if (c <= 256) softmax_grad_warp_rows_scalar<8><<<wgrid, 256, 0, st>>>(y, dy, dx, rows, c);
    else if (c <= 512) softmax_grad_warp_rows_scalar<16><<<wgrid, 256, 0, st>>>(y, dy, dx, rows, c);
    else softmax_grad_warp_rows_scalar<32><<<wgrid, 256, 0, st>>>(y, dy, dx, rows, c);
    return done();
  }
  const int grid = (int)(rows < 148 * 16 ? rows : 148 * 16);
  softmax_grad_rows<<<grid, cols >= 1024 ? 256 : 128, 0, st>>>(y, dy, dx, rows, cols);
  return done();
}

// y = softmax(scale * x + key-padding mask [+ causal mask]) row-wise; rows = batch * rows_per_batch, query index
// of a row = row % tq.  cols <= 1024 (TSB_ERR_UNSUPPORTED beyond: the caller composes the operators instead).
int tsb_masked_softmax(const float* x, const float* key_tokens, float* y, long long rows, long long cols,
                       long long rows_per_batch, int tq, float scale, int causal, void* stream) {
  if (rows <= 0 || cols <= 0 || rows_per_batch <= 0 || tq <= 0) return TSB_ERR_ARG;
  if (cols > 1024 || rows >= (1ll << 31) || rows_per_batch >= (1ll << 31)) return TSB_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long blocks = (rows + 7) / 8;
  const int wgrid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
  const int c = (int)cols;
  if (c % 4 == 0 && aligned16(x) && aligned16(y) && (!key_tokens || aligned16(key_tokens))) {
    const int nvec = c / 4;
    const float4* xv = reinterpret_cast<const float4*>(x);
    const float4* kv = reinterpret_cast<const float4*>(key_tokens);
    float4* yv = reinterpret_cast<float4*>(y);
#define TSB_MSV(NV) masked_softmax_warp_rows_v4<NV><<<wgrid, 256, 0, st>>>(xv, kv, yv, rows, nvec, rows_per_batch, tq, scale, causal)
    if (nvec <= 32) TSB_MSV(1);
    else if (nvec <= 64) TSB_MSV(2);
    else if (nvec <= 128) TSB_MSV(4);
    else TSB_MSV(8);
#undef TSB_MSV
    return done();
  }
#define TSB_MSM(NE) masked_softmax_warp_rows<NE><<<wgrid, 256, 0, st>>>(x, key_tokens, y, rows, c, rows_per_batch, tq, scale, causal)
  if (c <= 64) TSB_MSM(2);
  else if (c <= 128) TSB_MSM(4);
  else if (c <= 256) TSB_MSM(8);
  else if (c <= 512) TSB_MSM(16);
  else TSB_MSM(32);
#undef TSB_MSM
  return done();
}

int tsb_scaled_softmax_grad(const float* y, const float* dy, float* dx, long long rows, long long cols, float scale,
                            void* stream) {
  if (rows <= 0 || cols <= 0) return TSB_ERR_ARG;
  if (cols > 1024) return TSB_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long blocks = (rows + 7) / 8;
  const int wgrid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
  const int c = (int)cols;
  if (c % 4 == 0 && aligned16(y) && aligned16(dy) && aligned16(dx)) {
    const int nvec = c / 4;
    const float4* yv = reinterpret_cast<const float4*>(y);
    const float4* gv = reinterpret_cast<const float4*>(dy);
    float4* dv = reinterpret_cast<float4*>(dx);
#define TSB_SSV(NV) scaled_softmax_grad_warp_rows_v4<NV><<<wgrid, 256, 0, st>>>(yv, gv, dv, rows, nvec, scale)
    if (nvec <= 32) TSB_SSV(1);
    else if (nvec <= 64) TSB_SSV(2);
    else if (nvec <= 128) TSB_SSV(4);
    else TSB_SSV(8);
#undef TSB_SSV
    return done();
  }
#define TSB_SSG(NE) scaled_softmax_grad_warp_rows<NE><<<wgrid, 256, 0, st>>>(y, dy, dx, rows, c, scale)
  if (c <= 64) TSB_SSG(2);
  else if (c <= 128) TSB_SSG(4);
  else if (c <= 256) TSB_SSG(8);
  else if (c <= 512) TSB_SSG(16);
  else TSB_SSG(32);
#undef TSB_SSG
  return done();
}

int tsb_softmax_ce(const float* x, const float* labels, float* loss, long long rows, long long cols, void* stream) {
  if (rows <= 0 || cols <= 0) return TSB_ERR_ARG;
  float* rl = row_scratch(rows);
  if (!rl) return TSB_ERR_OOM;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = (int)(rows < 148 * 16 ? rows : 148 * 16);
  if (cols >= 512 && cols % 4 == 0 && cols / 4 < (1ll << 30) && aligned16(x) && aligned16(labels)) {
    ce_rows_v4<<<grid, cols >= 8192 ? 512 : 256, 0, st>>>(reinterpret_cast<const float4*>(x),
                                                         reinterpret_cast<const float4*>(labels), rl, rows,
                                                         (int)(cols / 4));
    mean_rows<<<1, 1024, 0, st>>>(rl, loss, rows);
    return done();
  }
  ce_rows<<<grid, cols >= 1024 ? 256 : 128, 0, st>>>(x, labels, rl, rows, cols);
  mean_rows<<<1, 1024, 0, st>>>(rl, loss, rows);
  return done();
}

int tsb_softmax_ce_grad(const float* x, const float* labels, const float* g, float* dx, long long rows,
                        long long cols, void* stream) {
  if (rows <= 0 || cols <= 0) return TSB_ERR_ARG;
  const int grid = (int)(rows < 148 * 16 ? rows : 148 * 16);
  if (cols >= 512 && cols % 4 == 0 && cols / 4 < (1ll << 30) && aligned16(x) && aligned16(labels) && aligned16(dx)) {
    ce_grad_rows_v4<<<grid, cols >= 8192 ? 512 : 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(x), reinterpret_cast<const float4*>(labels), g,
        reinterpret_cast<float4*>(dx), rows, (int)(cols / 4));
    return done();
  }
  ce_grad_rows<<<grid, cols >= 1024 ? 256 : 128, 0, static_cast<cudaStream_t>(stream)>>>(x, labels, g, dx, rows,
                                                                                         cols);
  return done();
}

}  // extern "C"
