// Host (CPU) operator library: OpenMP kernels for the operators a CPU-only run
// spends its time in.  Capability parity with the reference's oneDNN / OpenMP
// backend (src/dnnl_ops/*.cpp: matmul, element-wise, conv, pooling, batch-norm,
// softmax cross-entropy, optimizers); plain C++ here, since oneDNN is not part of
// this build.  Row-major fp32 throughout.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {

// C[m,n] = op(A) * op(B); lda/ldb are the row strides of the STORED matrices.
int tsb_cpu_matmul(const float* a, const float* b, float* c, int m, int n, int k, int trans_a, int trans_b) {
  const int lda = trans_a ? m : k, ldb = trans_b ? k : n;
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i) {
    float* crow = c + (int64_t)i * n;
    std::fill(crow, crow + n, 0.f);
    for (int p = 0; p < k; ++p) {
      const float av = trans_a ? a[(int64_t)p * lda + i] : a[(int64_t)i * lda + p];
      if (!trans_b) {
        const float* brow = b + (int64_t)p * ldb;
        for (int j = 0; j < n; ++j) crow[j] += av * brow[j];
      } else {
        for (int j = 0; j < n; ++j) crow[j] += av * b[(int64_t)j * ldb + p];
      }
    }
  }
  return 0;
}

// op: 0 add, 1 mul, 2 div, 3 relu_grad(x, g)
int tsb_cpu_binary(int op, const float* a, const float* b, float* y, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    switch (op) {
      case 0: y[i] = a[i] + b[i]; break;
      case 1: y[i] = a[i] * b[i]; break;
      case 2: y[i] = a[i] / b[i]; break;
      default: y[i] = a[i] > 0.f ? b[i] : (a[i] == 0.f ? 0.5f * b[i] : 0.f);
    }
  }
  return 0;
}

// op: 1 relu, 2 sigmoid, 3 tanh, 4 sqrt, 5 rsqrt, 6 neg, 7 add const, 8 mul const, 9 const / x
int tsb_cpu_unary(int op, const float* x, float* y, int64_t n, float alpha) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float v = x[i];
    switch (op) {
      case 1: y[i] = v > 0.f ? v : 0.f; break;
      case 2: y[i] = 1.f / (1.f + std::exp(-v)); break;
      case 3: y[i] = std::tanh(v); break;
      case 4: y[i] = std::sqrt(v); break;
      case 5: y[i] = 1.f / std::sqrt(v); break;
      case 6: y[i] = -v; break;
      case 7: y[i] = v + alpha; break;
      case 8: y[i] = v * alpha; break;
      case 9: y[i] = alpha / v; break;
      default: y[i] = v;
    }
  }
  return 0;
}

// NCHW x OIHW cross-correlation.
int tsb_cpu_conv2d(const float* x, const float* w, float* y, int N, int C, int H, int W, int O, int KH, int KW, int ph,
                   int pw, int stride) {
  const int OH = (H + 2 * ph - KH) / stride + 1, OW = (W + 2 * pw - KW) / stride + 1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; ++n)
    for (int o = 0; o < O; ++o) {
      float* yo = y + ((int64_t)n * O + o) * OH * OW;
      std::fill(yo, yo + (int64_t)OH * OW, 0.f);
      for (int c = 0; c < C; ++c) {
        const float* xc = x + ((int64_t)n * C + c) * H * W;
        const float* wc = w + ((int64_t)o * C + c) * KH * KW;
        for (int kh = 0; kh < KH; ++kh)
          for (int kw = 0; kw < KW; ++kw) {
            const float wv = wc[kh * KW + kw];
            for (int oh = 0; oh < OH; ++oh) {
              const int ih = oh * stride - ph + kh;
              if (ih < 0 || ih >= H) continue;
              for (int ow = 0; ow < OW; ++ow) {
                const int iw = ow * stride - pw + kw;
                if (iw < 0 || iw >= W) continue;
                yo[oh * OW + ow] += wv * xc[ih * W + iw];
              }
            }
          }
      }
    }
  return 0;
}

// kind 0 max, 1 average (count includes padding); NCHW.
int tsb_cpu_pool2d(int kind, const float* x, float* y, int N, int C, int H, int W, int KH, int KW, int pad, int stride) {
  const int OH = (H + 2 * pad - KH) / stride + 1, OW = (W + 2 * pad - KW) / stride + 1;
#pragma omp parallel for schedule(static)
  for (int64_t nc = 0; nc < (int64_t)N * C; ++nc) {
    const float* xc = x + nc * H * W;
    float* yc = y + nc * OH * OW;
    for (int oh = 0; oh < OH; ++oh)
      for (int ow = 0; ow < OW; ++ow) {
        float acc = kind == 0 ? -INFINITY : 0.f;
        for (int kh = 0; kh < KH; ++kh)
          for (int kw = 0; kw < KW; ++kw) {
            const int ih = oh * stride - pad + kh, iw = ow * stride - pad + kw;
            if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
            const float v = xc[ih * W + iw];
            acc = kind == 0 ? std::max(acc, v) : acc + v;
          }
        yc[oh * OW + ow] = kind == 0 ? acc : acc / (float)(KH * KW);
      }
  }
  return 0;
}

// Spatial batch-norm forward, NCHW; writes mean / invstd [C].
int tsb_cpu_batchnorm(const float* x, const float* scale, const float* bias, float* y, float* mean, float* invstd, int N,
                      int C, int HW, float eps) {
#pragma omp parallel for schedule(static)
  for (int c = 0; c < C; ++c) {
    double s = 0, ss = 0;
    for (int n = 0; n < N; ++n) {
      const float* p = x + ((int64_t)n * C + c) * HW;
      for (int i = 0; i < HW; ++i) { s += p[i]; ss += (double)p[i] * p[i]; }
    }
    const double cnt = (double)N * HW, m = s / cnt;
    const double var = std::max(0.0, ss / cnt - m * m);
    const float is = (float)(1.0 / std::sqrt(var + eps));
    mean[c] = (float)m; invstd[c] = is;
    for (int n = 0; n < N; ++n) {
      const float* p = x + ((int64_t)n * C + c) * HW;
      float* q = y + ((int64_t)n * C + c) * HW;
      for (int i = 0; i < HW; ++i) q[i] = (p[i] - (float)m) * is * scale[c] + bias[c];
    }
  }
  return 0;
}

// loss[0] = mean over rows of -sum(labels * log_softmax(logits)); dx optional = (softmax - labels) / rows.
int tsb_cpu_softmax_ce(const float* logits, const float* labels, float* loss, float* dx, int64_t rows, int64_t cols) {
  double total = 0;
#pragma omp parallel for reduction(+ : total) schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = logits + r * cols;
    const float* lr = labels + r * cols;
    float m = xr[0];
    for (int64_t i = 1; i < cols; ++i) m = std::max(m, xr[i]);
    double s = 0;
    for (int64_t i = 0; i < cols; ++i) s += std::exp((double)xr[i] - m);
    const double lse = m + std::log(s);
    double l = 0;
    for (int64_t i = 0; i < cols; ++i) {
      l -= lr[i] * (xr[i] - lse);
      if (dx) dx[r * cols + i] = (float)((std::exp(xr[i] - lse) - lr[i]) / (double)rows);
    }
    total += l;
  }
  loss[0] = (float)(total / (double)rows);
  return 0;
}

// kind: 0 sgd, 1 momentum, 2 nesterov, 3 adagrad, 4 adam; hyper as in the GPU kernel.
int tsb_cpu_optimizer(int kind, float* p, const float* g, float* s1, float* s2, int64_t n, const float* h) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float gi = g[i];
    switch (kind) {
      case 0: p[i] -= h[0] * gi; break;
      case 1: s1[i] = h[1] * s1[i] - h[0] * gi; p[i] += s1[i]; break;
      case 2: { const float lr_g = -h[0] * gi; s1[i] = h[1] * (s1[i] + lr_g); p[i] += s1[i] + lr_g; break; }
      case 3: s1[i] += gi * gi; p[i] -= h[0] * gi / (std::sqrt(s1[i]) + h[1]); break;
      default: {
        s1[i] = h[1] * s1[i] + (1.f - h[1]) * gi;
        s2[i] = h[2] * s2[i] + (1.f - h[2]) * gi * gi;
        p[i] -= h[0] * (s1[i] / (1.f - h[3])) / (std::sqrt(s2[i] / (1.f - h[4])) + h[5]);
      }
    }
  }
  return 0;
}


// ---------------------------------------------------------------------------------------------------------
// Backward and data-movement operators (the rest of the reference's host backend: src/dnnl_ops/Conv2d.cpp
// gradients, MaxPool / AvgPool gradients, BatchNorm gradient, Relu gradient, Softmax, Concat, Pad, Dropout,
// broadcast_to, ReduceSumAxisZero, Transpose, ArraySet).
// ---------------------------------------------------------------------------------------------------------

// dx[N,C,H,W] = data gradient of the NCHW x OIHW cross-correlation; dy[N,O,OH,OW].
int tsb_cpu_conv2d_dgrad(const float* dy, const float* w, float* dx, int N, int C, int H, int W, int O, int KH, int KW,
                         int OH, int OW, int ph, int pw, int stride) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c) {
      float* xc = dx + ((int64_t)n * C + c) * H * W;
      std::fill(xc, xc + (int64_t)H * W, 0.f);
      for (int o = 0; o < O; ++o) {
        const float* yo = dy + ((int64_t)n * O + o) * OH * OW;
        const float* wc = w + ((int64_t)o * C + c) * KH * KW;
        for (int kh = 0; kh < KH; ++kh)
          for (int kw = 0; kw < KW; ++kw) {
            const float wv = wc[kh * KW + kw];
            for (int oh = 0; oh < OH; ++oh) {
              const int ih = oh * stride - ph + kh;
              if (ih < 0 || ih >= H) continue;
              for (int ow = 0; ow < OW; ++ow) {
                const int iw = ow * stride - pw + kw;
                if (iw < 0 || iw >= W) continue;
                xc[ih * W + iw] += wv * yo[oh * OW + ow];
              }
            }
          }
      }
    }
  return 0;
}

// dw[O,C,KH,KW] = filter gradient.
int tsb_cpu_conv2d_wgrad(const float* x, const float* dy, float* dw, int N, int C, int H, int W, int O, int KH, int KW,
                         int OH, int OW, int ph, int pw, int stride) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int o = 0; o < O; ++o)
    for (int c = 0; c < C; ++c) {
      float* wc = dw + ((int64_t)o * C + c) * KH * KW;
      for (int kh = 0; kh < KH; ++kh)
        for (int kw = 0; kw < KW; ++kw) {
          double acc = 0;
          for (int n = 0; n < N; ++n) {
            const float* xc = x + ((int64_t)n * C + c) * H * W;
            const float* yo = dy + ((int64_t)n * O + o) * OH * OW;
            for (int oh = 0; oh < OH; ++oh) {
              const int ih = oh * stride - ph + kh;
              if (ih < 0 || ih >= H) continue;
              for (int ow = 0; ow < OW; ++ow) {
                const int iw = ow * stride - pw + kw;
                if (iw < 0 || iw >= W) continue;
                acc += (double)xc[ih * W + iw] * yo[oh * OW + ow];
              }
            }
          }
          wc[kh * KW + kw] = (float)acc;
        }
    }
  return 0;
}

// kind 0: max (the gradient goes to the first row-major maximum of each window; needs x), 1: average.
int tsb_cpu_pool2d_grad(int kind, const float* x, const float* dy, float* dx, int N, int C, int H, int W, int KH, int KW,
                        int OH, int OW, int pad, int stride) {
#pragma omp parallel for schedule(static)
  for (int64_t nc = 0; nc < (int64_t)N * C; ++nc) {
    const float* xc = x ? x + nc * H * W : nullptr;
    const float* gc = dy + nc * OH * OW;
    float* dc = dx + nc * H * W;
    std::fill(dc, dc + (int64_t)H * W, 0.f);
    for (int oh = 0; oh < OH; ++oh)
      for (int ow = 0; ow < OW; ++ow) {
        const float g = gc[oh * OW + ow];
        if (kind == 0) {
          // padding counts as -inf; the first maximum in row-major window order wins.  A window that lies
          // entirely in the padding has no element to give its gradient to.
          float best = -INFINITY;
          int bi = -1;
          for (int kh = 0; kh < KH; ++kh)
            for (int kw = 0; kw < KW; ++kw) {
              const int ih = oh * stride - pad + kh, iw = ow * stride - pad + kw;
              if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
              const float v = xc[ih * W + iw];
              if (bi < 0 || v > best) { best = v; bi = ih * W + iw; }
            }
          if (bi >= 0) dc[bi] += g;
        } else {
          const float share = g / (float)(KH * KW);
          for (int kh = 0; kh < KH; ++kh)
            for (int kw = 0; kw < KW; ++kw) {
              const int ih = oh * stride - pad + kh, iw = ow * stride - pad + kw;
              if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
              dc[ih * W + iw] += share;
            }
        }
      }
  }
  return 0;
}

// Spatial batch-norm backward, NCHW, from the saved mean / invstd.  relu != 0: dy is first masked by the sign of
// the forward output (scale * xhat + bias > 0), the fused BN+ReLU form.
int tsb_cpu_batchnorm_grad(const float* dy, const float* x, const float* scale, const float* bias, const float* mean,
                           const float* invstd, float* dx, float* dscale, float* dbias, int N, int C, int HW, int relu) {
#pragma omp parallel for schedule(static)
  for (int c = 0; c < C; ++c) {
    const float m = mean[c], is = invstd[c], sc = scale[c], bi = bias ? bias[c] : 0.f;
    double sg = 0, sgx = 0;
    for (int n = 0; n < N; ++n) {
      const float* g = dy + ((int64_t)n * C + c) * HW;
      const float* p = x + ((int64_t)n * C + c) * HW;
      for (int i = 0; i < HW; ++i) {
        const float xh = (p[i] - m) * is;
        const float gv = (relu && !(sc * xh + bi > 0.f)) ? 0.f : g[i];
        sg += gv; sgx += (double)gv * xh;
      }
    }
    const double cnt = (double)N * HW;
    if (dscale) dscale[c] = (float)sgx;
    if (dbias) dbias[c] = (float)sg;
    for (int n = 0; n < N; ++n) {
      const float* g = dy + ((int64_t)n * C + c) * HW;
      const float* p = x + ((int64_t)n * C + c) * HW;
      float* d = dx + ((int64_t)n * C + c) * HW;
      for (int i = 0; i < HW; ++i) {
        const float xh = (p[i] - m) * is;
        const float gv = (relu && !(sc * xh + bi > 0.f)) ? 0.f : g[i];
        d[i] = sc * is * (float)(gv - sg / cnt - xh * sgx / cnt);
      }
    }
  }
  return 0;
}

// dx = (softmax(logits) - labels) * g[0] / rows: the gradient of the mean cross-entropy, scaled by the incoming
// gradient of the loss (a one-element array).
int tsb_cpu_softmax_ce_grad(const float* logits, const float* labels, const float* g, float* dx, int64_t rows,
                            int64_t cols) {
  const double scale = (double)g[0] / (double)rows;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = logits + r * cols;
    const float* lr = labels + r * cols;
    float m = xr[0];
    for (int64_t i = 1; i < cols; ++i) m = std::max(m, xr[i]);
    double s = 0;
    for (int64_t i = 0; i < cols; ++i) s += std::exp((double)xr[i] - m);
    const double lse = m + std::log(s);
    for (int64_t i = 0; i < cols; ++i) dx[r * cols + i] = (float)((std::exp(xr[i] - lse) - lr[i]) * scale);
  }
  return 0;
}

int tsb_cpu_softmax(const float* x, float* y, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float* yr = y + r * cols;
    float m = xr[0];
    for (int64_t i = 1; i < cols; ++i) m = std::max(m, xr[i]);
    double s = 0;
    for (int64_t i = 0; i < cols; ++i) { yr[i] = std::exp(xr[i] - m); s += yr[i]; }
    const float inv = (float)(1.0 / s);
    for (int64_t i = 0; i < cols; ++i) yr[i] *= inv;
  }
  return 0;
}

// dx = y * (dy - sum(dy * y)) row-wise
int tsb_cpu_softmax_grad(const float* y, const float* dy, float* dx, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* yr = y + r * cols;
    const float* gr = dy + r * cols;
    double s = 0;
    for (int64_t i = 0; i < cols; ++i) s += (double)yr[i] * gr[i];
    for (int64_t i = 0; i < cols; ++i) dx[r * cols + i] = yr[i] * (gr[i] - (float)s);
  }
  return 0;
}

// y[cols] = sum over rows of x[rows][cols]
int tsb_cpu_reduce_sum_axis0(const float* x, float* y, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t j = 0; j < cols; ++j) {
    double s = 0;
    for (int64_t r = 0; r < rows; ++r) s += x[r * cols + j];
    y[j] = (float)s;
  }
  return 0;
}

// y[rows][cols] = x[cols] for every row
int tsb_cpu_broadcast_rows(const float* x, float* y, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) std::memcpy(y + r * cols, x, (size_t)cols * sizeof(float));
  return 0;
}

// y = transpose(x, perm): y's dimension d is x's dimension perm[d]; ndim <= 8.
int tsb_cpu_transpose(const float* x, float* y, int ndim, const int64_t* xshape, const int* perm) {
  if (ndim < 1 || ndim > 8) return 1;
  int64_t xstride[8], yshape[8], ystep[8], total = 1;
  xstride[ndim - 1] = 1;
  for (int d = ndim - 2; d >= 0; --d) xstride[d] = xstride[d + 1] * xshape[d + 1];
  for (int d = 0; d < ndim; ++d) { yshape[d] = xshape[perm[d]]; ystep[d] = xstride[perm[d]]; total *= yshape[d]; }
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < total; ++i) {
    int64_t rem = i, off = 0;
    for (int d = ndim - 1; d >= 0; --d) { off += (rem % yshape[d]) * ystep[d]; rem /= yshape[d]; }
    y[i] = x[off];
  }
  return 0;
}

// Copy a dense block: y[outer][ycols] columns [yoff, yoff + xcols) <- x[outer][xcols] (grad = 0), or the reverse
// direction x <- y (grad != 0).  Serves concat / concat gradient along any axis (outer = product of the leading
// dimensions, cols = product of the axis and the trailing ones) and pad / pad gradient of the last axes row by row.
int tsb_cpu_copy_block(float* x, float* y, int64_t outer, int64_t xcols, int64_t ycols, int64_t yoff, int grad) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < outer; ++r) {
    if (grad) std::memcpy(x + r * xcols, y + r * ycols + yoff, (size_t)xcols * sizeof(float));
    else std::memcpy(y + r * ycols + yoff, x + r * xcols, (size_t)xcols * sizeof(float));
  }
  return 0;
}

// Constant padding of the two trailing axes of x[outer][H][W] into y[outer][H + pt + pb][W + pl + pr] (grad = 0:
// y is written completely), or the gradient x <- interior of y (grad != 0).
int tsb_cpu_pad2d(float* x, float* y, int64_t outer, int H, int W, int pt, int pb, int pl, int pr, float value, int grad) {
  const int YH = H + pt + pb, YW = W + pl + pr;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < outer; ++r) {
    float* yr = y + r * YH * YW;
    float* xr = x + r * (int64_t)H * W;
    if (!grad) std::fill(yr, yr + (int64_t)YH * YW, value);
    for (int h = 0; h < H; ++h) {
      if (grad) std::memcpy(xr + (int64_t)h * W, yr + (int64_t)(h + pt) * YW + pl, (size_t)W * sizeof(float));
      else std::memcpy(yr + (int64_t)(h + pt) * YW + pl, xr + (int64_t)h * W, (size_t)W * sizeof(float));
    }
  }
  return 0;
}

int tsb_cpu_array_set(float* y, int64_t n, float value) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) y[i] = value;
  return 0;
}

// y = x * mask / keep; element i is kept when the 64-bit mix of (seed, i + offset) maps below `keep` — the same
// integer mix as the device kernel (csrc/kernels/misc_optim.cu: uniform01) and the NumPy path, so forward,
// recompute and backward of one step agree without storing the mask.
int tsb_cpu_dropout(const float* x, float* y, int64_t n, float keep, uint64_t seed, int64_t offset) {
  const float inv = 1.f / keep;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    uint64_t h = (uint64_t)(i + offset) + seed * 0x9E3779B97F4A7C15ull;
    h ^= h >> 30; h *= 0xBF58476D1CE4E5B9ull;
    h ^= h >> 27; h *= 0x94D049BB133111EBull;
    h ^= h >> 31;
    const float u = (float)(h >> 40) * (1.0f / 16777216.0f);
    y[i] = u < keep ? x[i] * inv : 0.f;
  }
  return 0;
}

}  // extern "C"
