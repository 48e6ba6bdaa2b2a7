// Element-wise, strided-copy and strided-reduce kernels (fp32).
//
// Flat variants move 16 bytes per thread per step with a grid sized to the SM
// count (HBM-bound: one read + one write per element).  Strided variants take
// the shape / stride tables as kernel parameters, so transpose, slice, concat,
// pad, the broadcast family and layout changes (NCHW <-> channels-last) are all
// one launch with no host-side table copies.
//
// Roles in the reference: src/ops/{Relu,AddConst,AddElewise,MultiplyConst,
// MultiplyElewise,DivideConst,DivideElewise,Opposite,Sqrt,Tanh,Sigmoid,ArraySet,
// Where,Transpose,Slice,Concat,Pad,Broadcast,BroadcastShape,ReduceSum,
// ReduceSumAxisZero,Conv2dBroadcast,Conv2dReduceSum}.cu
#include <cuda_runtime.h>
#include "scratch.h"
#include <stdint.h>

#define TSB_OK 0
#define TSB_ERR_ARG 1
#define TSB_ERR_UNSUPPORTED 2
#define TSB_ERR_LAUNCH 3

namespace {

enum { UN_COPY, UN_RELU, UN_SIGMOID, UN_TANH, UN_SQRT, UN_RSQRT, UN_NEG, UN_ADDC, UN_MULC, UN_CDIV, UN_FILL };
enum { BIN_ADD, BIN_MUL, BIN_DIV, BIN_RELU_GRAD, BIN_SUB, BIN_ADD_RELU, BIN_RELU_GRAD_OUT };

constexpr int MAXD = 8;
struct Dims {
  long long shape[MAXD];
  long long s0[MAXD];
  long long s1[MAXD];
  long long s2[MAXD];
  int nd;
  int small;   // the element count is below 2^32: index arithmetic may run in 32 bits
};

template <int OP>
__device__ __forceinline__ float un(float x, float a) {
  switch (OP) {
    case UN_COPY: return x;
    case UN_RELU: return fmaxf(x, 0.f);
    case UN_SIGMOID: return 1.f / (1.f + __expf(-x));
    case UN_TANH: return tanhf(x);
    case UN_SQRT: return sqrtf(x);
    case UN_RSQRT: return rsqrtf(x);
    case UN_NEG: return -x;
    case UN_ADDC: return x + a;
    case UN_MULC: return x * a;
    case UN_CDIV: return a / x;
    default: return a;   // UN_FILL
  }
}
template <int OP>
__device__ __forceinline__ float bin(float a, float b) {
  switch (OP) {
    case BIN_ADD: return a + b;
    case BIN_MUL: return a * b;
    case BIN_DIV: return a / b;
    case BIN_RELU_GRAD: return a > 0.f ? b : (a == 0.f ? 0.5f * b : 0.f);
    case BIN_ADD_RELU: return fmaxf(a + b, 0.f);              // residual add + ReLU in one pass
    case BIN_RELU_GRAD_OUT: return a > 0.f ? b : 0.f;         // a = the ReLU OUTPUT: gradient passes where it is positive
    default: return a - b;
  }
}

template <int OP>
__global__ void unary_flat(const float* __restrict__ x, float* __restrict__ y, long long n, float a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (vec) {
    const long long n4 = n >> 2;
    for (long long j = i; j < n4; j += stride) {
      float4 v = OP == UN_FILL ? make_float4(0, 0, 0, 0) : reinterpret_cast<const float4*>(x)[j];
      v.x = un<OP>(v.x, a); v.y = un<OP>(v.y, a); v.z = un<OP>(v.z, a); v.w = un<OP>(v.w, a);
      reinterpret_cast<float4*>(y)[j] = v;
    }
    for (long long j = (n4 << 2) + i; j < n; j += stride) y[j] = un<OP>(OP == UN_FILL ? 0.f : x[j], a);
  } else {
    for (; i < n; i += stride) y[i] = un<OP>(OP == UN_FILL ? 0.f : x[i], a);
  }
}

template <int OP>
__global__ void binary_flat(const float* __restrict__ p, const float* __restrict__ q, float* __restrict__ y,
                            long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(q) |
                     reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (vec) {
    const long long n4 = n >> 2;
    for (long long j = i; j < n4; j += stride) {
      const float4 a = reinterpret_cast<const float4*>(p)[j];
      const float4 b = reinterpret_cast<const float4*>(q)[j];
      float4 o;
      o.x = bin<OP>(a.x, b.x); o.y = bin<OP>(a.y, b.y); o.z = bin<OP>(a.z, b.z); o.w = bin<OP>(a.w, b.w);
      reinterpret_cast<float4*>(y)[j] = o;
    }
    for (long long j = (n4 << 2) + i; j < n; j += stride) y[j] = bin<OP>(p[j], q[j]);
  } else {
    for (; i < n; i += stride) y[i] = bin<OP>(p[i], q[i]);
  }
}

__global__ void where_flat(const float* __restrict__ c, const float* __restrict__ a, const float* __restrict__ b,
                           float* __restrict__ y, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = c[i] != 0.f ? a[i] : b[i];
}

// y[r, c] = x[r, c] + b[c] on a dense row-major [rows, cols] view, 16 bytes per thread (the bias of a
// dense layer added without materialising the broadcast).
__global__ void bias_add_v4(const float4* __restrict__ x, const float4* __restrict__ b, float4* __restrict__ y,
                            long long n4, unsigned cols4) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += stride) {
    const unsigned c = (n4 >> 32) == 0 ? (unsigned)i % cols4 : (unsigned)(i % cols4);
    const float4 v = x[i], w = __ldg(b + c);
    y[i] = make_float4(v.x + w.x, v.y + w.y, v.z + w.z, v.w + w.w);
  }
}

// index decomposition: the LAST dim varies fastest across threads
// (tensors of fewer than 2^32 elements are decomposed with 32-bit divisions, several times cheaper
// than 64-bit ones)
__device__ __forceinline__ void offsets2(const Dims& d, long long idx, long long& o0, long long& o1) {
  o0 = 0; o1 = 0;
  if (d.small) {
    unsigned r = (unsigned)idx;
#pragma unroll
    for (int k = MAXD - 1; k >= 0; --k) {
      if (k < d.nd) {
        const unsigned sh = (unsigned)d.shape[k];
        const unsigned q = r / sh;
        const long long c = r - q * sh;
        r = q;
        o0 += c * d.s0[k];
        o1 += c * d.s1[k];
      }
    }
    return;
  }
#pragma unroll
  for (int k = MAXD - 1; k >= 0; --k) {
    if (k < d.nd) {
      const long long c = idx % d.shape[k];
      idx /= d.shape[k];
      o0 += c * d.s0[k];
      o1 += c * d.s1[k];
    }
  }
}
__device__ __forceinline__ void offsets3(const Dims& d, long long idx, long long& o0, long long& o1,
                                         long long& o2) {
  o0 = 0; o1 = 0; o2 = 0;
  if (d.small) {
    unsigned r = (unsigned)idx;
#pragma unroll
    for (int k = MAXD - 1; k >= 0; --k) {
      if (k < d.nd) {
        const unsigned sh = (unsigned)d.shape[k];
        const unsigned q = r / sh;
        const long long c = r - q * sh;
        r = q;
        o0 += c * d.s0[k];
        o1 += c * d.s1[k];
        o2 += c * d.s2[k];
      }
    }
    return;
  }
#pragma unroll
  for (int k = MAXD - 1; k >= 0; --k) {
    if (k < d.nd) {
      const long long c = idx % d.shape[k];
      idx /= d.shape[k];
      o0 += c * d.s0[k];
      o1 += c * d.s1[k];
      o2 += c * d.s2[k];
    }
  }
}

// Strided copy whose innermost dimension is contiguous on both sides and a multiple of four floats
// (a channel range of a channels-last tensor: concat / slice along channels, padded feeds): the same
// index walk as unary_strided, but in units of 16 bytes.  `d` holds the shape and strides already
// divided by four in the innermost dimension / for the outer strides.
__global__ void copy_strided_v4(const float4* __restrict__ x, float4* __restrict__ y, const Dims d, long long n4) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += stride) {
    long long ox, oy;
    offsets2(d, i, ox, oy);
    y[oy] = x[ox];
  }
}

template <int OP>
__global__ void unary_strided(const float* __restrict__ x, float* __restrict__ y, const Dims d, long long n,
                              float a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    long long ox, oy;
    offsets2(d, i, ox, oy);
    y[oy] = un<OP>(OP == UN_FILL ? 0.f : x[ox], a);
  }
}

// 2-D tiled transpose-copy through shared memory for the common "two dims whose
// fast axis differs between source and destination" case (NCHW <-> NHWC,
// matrix transpose): both the read and the write are coalesced.
__global__ void copy_tiled(const float* __restrict__ x, float* __restrict__ y, long long outer, long long R,
                           long long Cc, long long xs_outer, long long xs_r, long long xs_c, long long ys_outer,
                           long long ys_r, long long ys_c) {
  // source is contiguous along c (xs_c == 1), destination along r (ys_r == 1)
  __shared__ float tile[32][33];
  const long long tiles_r = (R + 31) / 32, tiles_c = (Cc + 31) / 32;
  const long long per_outer = tiles_r * tiles_c;
  const long long total = outer * per_outer;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const long long o = t / per_outer;
    const long long tr = (t % per_outer) / tiles_c, tc = t % tiles_c;
    const long long r0 = tr * 32, c0 = tc * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
      const long long r = r0 + j, c = c0 + threadIdx.x;
      if (r < R && c < Cc) tile[j][threadIdx.x] = x[o * xs_outer + r * xs_r + c * xs_c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
      const long long c = c0 + j, r = r0 + threadIdx.x;
      if (r < R && c < Cc) y[o * ys_outer + r * ys_r + c * ys_c] = tile[threadIdx.x][j];
    }
    __syncthreads();
  }
}

template <int OP>
__global__ void binary_strided(const float* __restrict__ p, const float* __restrict__ q, float* __restrict__ y,
                               const Dims d, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    long long oa, ob, oy;
    offsets3(d, i, oa, ob, oy);
    y[oy] = bin<OP>(p[oa], q[ob]);
  }
}

// Row forms of the strided kernels for a long innermost dimension: a warp walks one row, so the outer
// index is decomposed once per row instead of once per element.  Block = 32 lanes x 8 rows.
template <int OP>
__global__ void binary_rows(const float* __restrict__ p, const float* __restrict__ q, float* __restrict__ y,
                            const Dims o, long long outer, int inner, long long sa, long long sb,
                            long long sy) {
  for (long long r = blockIdx.x * (long long)blockDim.y + threadIdx.y; r < outer;
       r += (long long)gridDim.x * blockDim.y) {
    long long oa, ob, oy;
    offsets3(o, r, oa, ob, oy);
    // gridDim.y column slices per row: few long rows would otherwise leave most SMs idle
    for (int c = threadIdx.x + 32 * blockIdx.y; c < inner; c += 32 * gridDim.y)
      y[oy + c * sy] = bin<OP>(p[oa + c * sa], q[ob + c * sb]);
  }
}
template <int OP>
__global__ void unary_rows(const float* __restrict__ x, float* __restrict__ y, const Dims o, long long outer,
                           int inner, float a, long long sx, long long sy) {
  for (long long r = blockIdx.x * (long long)blockDim.y + threadIdx.y; r < outer;
       r += (long long)gridDim.x * blockDim.y) {
    long long ox, oy;
    offsets2(o, r, ox, oy);
    for (int c = threadIdx.x + 32 * blockIdx.y; c < inner; c += 32 * gridDim.y)
      y[oy + c * sy] = un<OP>(OP == UN_FILL ? 0.f : x[ox + c * sx], a);
  }
}

// y[keep] = sum_red x[keep, red].  One warp per output element when the reduced
// extent is long, otherwise one thread.  Deterministic (fixed order + shuffles).
struct RDims {
  long long kshape[MAXD], kxs[MAXD], kys[MAXD];
  long long rshape[MAXD], rxs[MAXD];
  int nk, nr;
};
__global__ void reduce_sum_kernel(const float* __restrict__ x, float* __restrict__ y, const RDims d,
                                  long long nkeep, long long nred) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long o = warp; o < nkeep; o += nwarps) {
    long long idx = o, xo = 0, yo = 0;
    for (int k = d.nk - 1; k >= 0; --k) {
      const long long c = idx % d.kshape[k];
      idx /= d.kshape[k];
      xo += c * d.kxs[k];
      yo += c * d.kys[k];
    }
    float acc = 0.f;
    for (long long r = lane; r < nred; r += 32) {
      long long ridx = r, ro = 0;
      for (int k = d.nr - 1; k >= 0; --k) {
        const long long c = ridx % d.rshape[k];
        ridx /= d.rshape[k];
        ro += c * d.rxs[k];
      }
      acc += x[xo + ro];
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) y[yo] = acc;
  }
}

// Column sums of a row-major [rows, cols] view with cols contiguous (the
// "reduce over leading dims" case: bias gradients, axis-0 sums): coalesced along
// cols, two-stage and deterministic.
__global__ void colsum_partial(const float* __restrict__ x, float* __restrict__ part, long long rows,
                               long long cols, long long ld, int chunks) {
  const long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int ch = blockIdx.y;
  if (c >= cols) return;
  const long long per = (rows + chunks - 1) / chunks;
  const long long r0 = ch * per, r1 = min(rows, r0 + per);
  float acc = 0.f;
  for (long long r = r0; r < r1; ++r) acc += x[r * ld + c];
  part[(long long)ch * cols + c] = acc;
}
// 16-byte variant: a thread owns four adjacent columns and keeps four rows in flight.
__global__ void colsum_partial_v4(const float4* __restrict__ x, float4* __restrict__ part, long long rows,
                                  int cols4, long long ld4, int chunks) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int ch = blockIdx.y;
  if (c >= cols4) return;
  const long long per = (rows + chunks - 1) / chunks;
  const long long r0 = ch * per, r1 = min(rows, r0 + per);
  float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0, a2 = a0, a3 = a0;
  long long r = r0;
  for (; r + 3 < r1; r += 4) {
    const float4 v0 = __ldg(x + r * ld4 + c), v1 = __ldg(x + (r + 1) * ld4 + c), v2 = __ldg(x + (r + 2) * ld4 + c),
                 v3 = __ldg(x + (r + 3) * ld4 + c);
    a0.x += v0.x; a0.y += v0.y; a0.z += v0.z; a0.w += v0.w;
    a1.x += v1.x; a1.y += v1.y; a1.z += v1.z; a1.w += v1.w;
    a2.x += v2.x; a2.y += v2.y; a2.z += v2.z; a2.w += v2.w;
    a3.x += v3.x; a3.y += v3.y; a3.z += v3.z; a3.w += v3.w;
  }
  for (; r < r1; ++r) {
    const float4 v = __ldg(x + r * ld4 + c);
    a0.x += v.x; a0.y += v.y; a0.z += v.z; a0.w += v.w;
  }
  part[(long long)ch * cols4 + c] =
      make_float4((a0.x + a1.x) + (a2.x + a3.x), (a0.y + a1.y) + (a2.y + a3.y), (a0.z + a1.z) + (a2.z + a3.z),
                  (a0.w + a1.w) + (a2.w + a3.w));
}
// Second stage for many chunks: 32 columns x 8 chunk lanes per block, lanes joined in a fixed order.
__global__ void colsum_final_lanes(const float* __restrict__ part, float* __restrict__ y, long long cols, int chunks,
                                   long long ys) {
  __shared__ float sh[8][33];
  const long long c = blockIdx.x * 32ll + threadIdx.x;
  float acc = 0.f;
  if (c < cols)
    for (int ch = threadIdx.y; ch < chunks; ch += 8) acc += part[(long long)ch * cols + c];
  sh[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) t += sh[j][threadIdx.x];
    y[c * ys] = t;
  }
}
__global__ void colsum_final(const float* __restrict__ part, float* __restrict__ y, long long cols, int chunks,
                             long long ys) {
  const long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float acc = 0.f;
  for (int ch = 0; ch < chunks; ++ch) acc += part[(long long)ch * cols + c];
  y[c * ys] = acc;
}

int grid_for(long long work_items, int threads) {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = (long long)sms * 8;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}

int done() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

float* colsum_scratch() {   // 64 chunks x up to 64K columns
  return static_cast<float*>(tsb_scratch::get(nullptr, tsb_scratch::COLSUM_PARTIALS, 64ull * 65536 * 4));
}

}  // namespace

// Grid of the row-form kernels: eight rows per block along x; when that leaves SMs idle (few long rows, e.g. an
// NCHW image batch seen as N * C rows of H * W), the columns of a row are cut into gridDim.y slices of >= 256.
dim3 rows_grid(long long outer, int inner) {
  const int gx = grid_for(outer * 32, 256);
  int gy = 1;
  const int want = 148 * 4;
  if (gx < want) {
    gy = (want + gx - 1) / gx;
    const int most = (inner + 255) / 256;
    if (gy > most) gy = most;
    if (gy < 1) gy = 1;
    if (gy > 65535) gy = 65535;
  }
  return dim3((unsigned)gx, (unsigned)gy, 1);
}

#define UN_CASE(OPC) \
  case OPC: unary_flat<OPC><<<grid, 256, 0, st>>>(x, y, n, alpha); break;
#define UNR_CASE(OPC) \
  case OPC: unary_rows<OPC><<<rgrid, dim3(32, 8), 0, st>>>(x, y, dr, outer, inner, alpha, xs[nd - 1], ys[nd - 1]); break;
#define BINR_CASE(OPC) \
  case OPC: binary_rows<OPC><<<rgrid, dim3(32, 8), 0, st>>>(a, b, y, dr, outer, inner, as[nd - 1], bs[nd - 1], ys[nd - 1]); break;
#define UNS_CASE(OPC) \
  case OPC: unary_strided<OPC><<<grid, 256, 0, st>>>(x, y, d, n, alpha); break;
#define BIN_CASE(OPC) \
  case OPC: binary_flat<OPC><<<grid, 256, 0, st>>>(a, b, y, n); break;
#define BINS_CASE(OPC) \
  case OPC: binary_strided<OPC><<<grid, 256, 0, st>>>(a, b, y, d, n); break;

extern "C" {

int tsb_ew_unary(int op, const float* x, float* y, long long n, float alpha, void* stream) {
  if (n <= 0) return TSB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for((n + 3) / 4, 256);
  switch (op) {
    UN_CASE(UN_COPY) UN_CASE(UN_RELU) UN_CASE(UN_SIGMOID) UN_CASE(UN_TANH) UN_CASE(UN_SQRT) UN_CASE(UN_RSQRT)
    UN_CASE(UN_NEG) UN_CASE(UN_ADDC) UN_CASE(UN_MULC) UN_CASE(UN_CDIV) UN_CASE(UN_FILL)
    default: return TSB_ERR_ARG;
  }
  return done();
}

int tsb_ew_binary(int op, const float* a, const float* b, float* y, long long n, void* stream) {
  if (n <= 0) return TSB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for((n + 3) / 4, 256);
  switch (op) {
    BIN_CASE(BIN_ADD) BIN_CASE(BIN_MUL) BIN_CASE(BIN_DIV) BIN_CASE(BIN_RELU_GRAD) BIN_CASE(BIN_SUB)
    BIN_CASE(BIN_ADD_RELU) BIN_CASE(BIN_RELU_GRAD_OUT)
    default: return TSB_ERR_ARG;
  }
  return done();
}

int tsb_where(const float* c, const float* a, const float* b, float* y, long long n, void* stream) {
  if (n <= 0) return TSB_OK;
  where_flat<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(c, a, b, y, n);
  return done();
}

int tsb_strided_unary(int op, const float* x, float* y, int nd, const long long* shape, const long long* xs,
                      const long long* ys, float alpha, void* stream) {
  if (nd < 1 || nd > MAXD) return TSB_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Dims d;
  d.nd = nd;
  long long n = 1;
  for (int i = 0; i < nd; ++i) { d.shape[i] = shape[i]; d.s0[i] = xs[i]; d.s1[i] = ys[i]; d.s2[i] = 0; n *= shape[i]; }
  if (n <= 0) return TSB_OK;
  d.small = n < (1ll << 32);
  // 16-byte path: some dimension is contiguous on both sides (the channel range of a channels-last
  // tensor given in logical N, C, H, W order) and everything is a multiple of four floats.  The order
  // of the dimensions does not matter to a copy, so that dimension is moved last.
  if (op == UN_COPY && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
    int cd = -1;
    for (int i = nd - 1; i >= 0; --i)
      if (xs[i] == 1 && ys[i] == 1 && (shape[i] & 3) == 0) { cd = i; break; }
    bool ok = cd >= 0;
    for (int i = 0; i < nd && ok; ++i)
      if (i != cd) ok = (xs[i] & 3) == 0 && (ys[i] & 3) == 0;
    if (ok) {
      Dims v = d;
      // rotate dimension cd to the end
      for (int i = cd; i + 1 < nd; ++i) {
        v.shape[i] = d.shape[i + 1]; v.s0[i] = d.s0[i + 1]; v.s1[i] = d.s1[i + 1];
      }
      v.shape[nd - 1] = shape[cd] / 4; v.s0[nd - 1] = 1; v.s1[nd - 1] = 1;
      for (int i = 0; i < nd - 1; ++i) { v.s0[i] /= 4; v.s1[i] /= 4; }
      const long long n4 = n / 4;
      copy_strided_v4<<<grid_for(n4, 256), 256, 0, st>>>(reinterpret_cast<const float4*>(x),
                                                          reinterpret_cast<float4*>(y), v, n4);
      return done();
    }
  }
  // coalesced tiled path: copy where src is contiguous along the last dim and dst along another one
  if (op == UN_COPY && nd >= 2 && nd <= 3 && xs[nd - 1] == 1 && ys[nd - 1] != 1) {
    int rdim = -1;
    for (int i = 0; i < nd - 1; ++i) if (ys[i] == 1) rdim = i;
    if (rdim >= 0 && shape[rdim] >= 8 && shape[nd - 1] >= 8) {
      long long outer = 1, xso = 0, yso = 0;
      if (nd == 3) { const int od = rdim == 0 ? 1 : 0; outer = shape[od]; xso = xs[od]; yso = ys[od]; }
      const long long tiles = outer * ((shape[rdim] + 31) / 32) * ((shape[nd - 1] + 31) / 32);
      int grid = tiles > 148ll * 16 ? 148 * 16 : (int)tiles;
      copy_tiled<<<grid, dim3(32, 8), 0, st>>>(x, y, outer, shape[rdim], shape[nd - 1], xso, xs[rdim], 1, yso, 1,
                                               ys[nd - 1]);
      return done();
    }
  }
  if (op == UN_COPY && nd >= 2 && nd <= 3 && ys[nd - 1] == 1 && xs[nd - 1] != 1) {
    int cdim = -1;   // the dim along which the source is contiguous
    for (int i = 0; i < nd - 1; ++i) if (xs[i] == 1) cdim = i;
    if (cdim >= 0 && shape[cdim] >= 8 && shape[nd - 1] >= 8) {
      long long outer = 1, xso = 0, yso = 0;
      if (nd == 3) { const int od = cdim == 0 ? 1 : 0; outer = shape[od]; xso = xs[od]; yso = ys[od]; }
      // roles: r = last dim (dst-contiguous), c = cdim (src-contiguous)
      const long long tiles = outer * ((shape[nd - 1] + 31) / 32) * ((shape[cdim] + 31) / 32);
      int grid = tiles > 148ll * 16 ? 148 * 16 : (int)tiles;
      copy_tiled<<<grid, dim3(32, 8), 0, st>>>(x, y, outer, shape[nd - 1], shape[cdim], xso, xs[nd - 1], 1, yso, 1,
                                               ys[cdim]);
      return done();
    }
  }
  if (nd >= 2 && shape[nd - 1] >= 64 && shape[nd - 1] < (1ll << 31)) {
    const long long outer = n / shape[nd - 1];
    const int inner = (int)shape[nd - 1];
    const dim3 rgrid = rows_grid(outer, inner);
    Dims dr = d;
    dr.nd = nd - 1;
    switch (op) {
      UNR_CASE(UN_COPY) UNR_CASE(UN_RELU) UNR_CASE(UN_SIGMOID) UNR_CASE(UN_TANH) UNR_CASE(UN_SQRT)
      UNR_CASE(UN_RSQRT) UNR_CASE(UN_NEG) UNR_CASE(UN_ADDC) UNR_CASE(UN_MULC) UNR_CASE(UN_CDIV) UNR_CASE(UN_FILL)
      default: return TSB_ERR_ARG;
    }
    return done();
  }
  const int grid = grid_for(n, 256);
  switch (op) {
    UNS_CASE(UN_COPY) UNS_CASE(UN_RELU) UNS_CASE(UN_SIGMOID) UNS_CASE(UN_TANH) UNS_CASE(UN_SQRT)
    UNS_CASE(UN_RSQRT) UNS_CASE(UN_NEG) UNS_CASE(UN_ADDC) UNS_CASE(UN_MULC) UNS_CASE(UN_CDIV) UNS_CASE(UN_FILL)
    default: return TSB_ERR_ARG;
  }
  return done();
}

int tsb_bias_add(const float* x, const float* b, float* y, long long rows, long long cols, void* stream) {
  if (rows <= 0 || cols <= 0) return TSB_OK;
  if ((cols & 3) || cols >= (1ll << 32) ||
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(y)) & 15))
    return TSB_ERR_UNSUPPORTED;
  const long long n4 = rows * (cols / 4);
  bias_add_v4<<<grid_for(n4, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(x), reinterpret_cast<const float4*>(b), reinterpret_cast<float4*>(y), n4,
      (unsigned)(cols / 4));
  return done();
}

int tsb_strided_binary(int op, const float* a, const float* b, float* y, int nd, const long long* shape,
                       const long long* as, const long long* bs, const long long* ys, void* stream) {
  if (nd < 1 || nd > MAXD) return TSB_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Dims d;
  d.nd = nd;
  long long n = 1;
  for (int i = 0; i < nd; ++i) { d.shape[i] = shape[i]; d.s0[i] = as[i]; d.s1[i] = bs[i]; d.s2[i] = ys[i]; n *= shape[i]; }
  if (n <= 0) return TSB_OK;
  d.small = n < (1ll << 32);
  if (nd >= 2 && shape[nd - 1] >= 64 && shape[nd - 1] < (1ll << 31)) {
    const long long outer = n / shape[nd - 1];
    const int inner = (int)shape[nd - 1];
    const dim3 rgrid = rows_grid(outer, inner);
    Dims dr = d;
    dr.nd = nd - 1;
    switch (op) {
      BINR_CASE(BIN_ADD) BINR_CASE(BIN_MUL) BINR_CASE(BIN_DIV) BINR_CASE(BIN_RELU_GRAD) BINR_CASE(BIN_SUB)
      BINR_CASE(BIN_ADD_RELU) BINR_CASE(BIN_RELU_GRAD_OUT)
      default: return TSB_ERR_ARG;
    }
    return done();
  }
  const int grid = grid_for(n, 256);
  switch (op) {
    BINS_CASE(BIN_ADD) BINS_CASE(BIN_MUL) BINS_CASE(BIN_DIV) BINS_CASE(BIN_RELU_GRAD) BINS_CASE(BIN_SUB)
    BINS_CASE(BIN_ADD_RELU) BINS_CASE(BIN_RELU_GRAD_OUT)
    default: return TSB_ERR_ARG;
  }
  return done();
}

int tsb_reduce_sum(const float* x, float* y, int nk, const long long* kshape, const long long* kxs,
                   const long long* kys, int nr, const long long* rshape, const long long* rxs, void* stream) {
  if (nk < 1 || nk > MAXD || nr < 1 || nr > MAXD) return TSB_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RDims d;
  d.nk = nk; d.nr = nr;
  long long nkeep = 1, nred = 1;
  for (int i = 0; i < nk; ++i) { d.kshape[i] = kshape[i]; d.kxs[i] = kxs[i]; d.kys[i] = kys[i]; nkeep *= kshape[i]; }
  for (int i = 0; i < nr; ++i) { d.rshape[i] = rshape[i]; d.rxs[i] = rxs[i]; nred *= rshape[i]; }
  if (nkeep <= 0) return TSB_OK;
  // fast path: kept dims collapse to one contiguous column index and the reduced
  // dims to one row index with a constant stride (e.g. [rows, cols] -> [cols])
  if (nk == 1 && nr == 1 && kxs[0] == 1 && nkeep <= 65536 && nred >= 64) {
    float* part = colsum_scratch();
    if (part) {
      if ((nkeep & 3) == 0 && (rxs[0] & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        // scratch: 64 x 65536 floats, so up to 256 chunks for 16384 columns or fewer
        long long cmax = (64ll * 65536) / nkeep;
        if (cmax > 256) cmax = 256;
        long long want = nred / 32;
        if (want < 1) want = 1;
        const int chunks = (int)(want < cmax ? want : cmax);
        const int cols4 = (int)(nkeep / 4);
        dim3 g1((unsigned)((cols4 + 127) / 128), chunks);
        colsum_partial_v4<<<g1, 128, 0, st>>>(reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(part),
                                              nred, cols4, rxs[0] / 4, chunks);
        colsum_final_lanes<<<(unsigned)((nkeep + 31) / 32), dim3(32, 8), 0, st>>>(part, y, nkeep, chunks, kys[0]);
        return done();
      }
      int chunks = (int)(nred / 64 < 64 ? (nred / 64 < 1 ? 1 : nred / 64) : 64);
      dim3 g1((unsigned)((nkeep + 127) / 128), chunks);
      colsum_partial<<<g1, 128, 0, st>>>(x, part, nred, nkeep, rxs[0], chunks);
      colsum_final<<<(unsigned)((nkeep + 127) / 128), 128, 0, st>>>(part, y, nkeep, chunks, kys[0]);
      return done();
    }
  }
  const int grid = grid_for(nkeep * 32, 256);
  reduce_sum_kernel<<<grid, 256, 0, st>>>(x, y, d, nkeep, nred);
  return done();
}

}  // extern "C"
