"""Python entry points of the host operator library (role of the reference's
``python/athena/cpu_links/dnnl_op.py:8-274``): one thin function per C entry of
``csrc/runtime/cpu_ops.cc`` operating on contiguous fp32 NumPy arrays.  Executors on a
CPU context (``ndarray.cpu``) call them through ``Op.cpu_compute``: matrix products, convolution and
its two gradients, pooling and its gradients, batch norm forward / backward, the element-wise family,
soft-max (+ gradient), soft-max cross-entropy, concat / pad (+ gradients), transpose, broadcast,
reduce-sum over axis 0, fills, dropout, optimizers.  Operators without a native kernel, and ``ctx=None``
(the NumPy oracle), use NumPy."""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p

import numpy as np

from . import _base


def _p(a):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return c_void_p(a.ctypes.data)


_RT = []


def _rt():
    """The host library behind the recording proxy: a CPU-context step can be recorded as a list of native calls
    and replayed by the C++ loop like a GPU step (``runtime/tape.py``)."""
    if not _RT:
        from .utils.launch_counter import CountingLib
        _RT.append(CountingLib(_base.runtime(), count=False))
    return _RT[0]


#: native kernel calls made so far (tests check that a CPU-context run really goes through the library)
CALLS = [0]


def ok(*arrays):
    """The native kernels take C-contiguous fp32 NumPy arrays."""
    return all(isinstance(a, np.ndarray) and a.dtype == np.float32 and a.flags.c_contiguous for a in arrays)


#: operator name -> code of tsb_cpu_unary / tsb_cpu_binary
UNARY = {"Relu": 1, "Sigmoid": 2, "Tanh": 3, "Sqrt": 4, "Rsqrt": 5, "Opposite": 6, "AddConst": 7, "MulConst": 8,
         "DivConst": 9}
BINARY = {"Add": 0, "Mul": 1, "Div": 2, "ReluGradient": 3}


def matrix_multiply(a, b, c, trans_a=False, trans_b=False):
    CALLS[0] += 1
    m, n = c.shape
    k = a.shape[0] if trans_a else a.shape[1]
    _rt().tsb_cpu_matmul(_p(a), _p(b), _p(c), m, n, k, int(trans_a), int(trans_b))


def binary(op, a, b, y):
    CALLS[0] += 1
    _rt().tsb_cpu_binary(c_int(op), _p(a), _p(b), _p(y), c_int64(y.size))


def unary(op, x, y, alpha=0.0):
    CALLS[0] += 1
    _rt().tsb_cpu_unary(c_int(op), _p(x), _p(y), c_int64(y.size), c_float(alpha))


def conv2d(x, w, y, padding=0, padding2=None, stride=1):
    CALLS[0] += 1
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    pw = padding if padding2 is None else padding2
    _rt().tsb_cpu_conv2d(_p(x), _p(w), _p(y), n, c, h, wd, o, kh, kw, padding, pw, stride)


def pool2d(kind, x, y, kh, kw, padding, stride):
    CALLS[0] += 1
    n, c, h, w = x.shape
    _rt().tsb_cpu_pool2d(kind, _p(x), _p(y), n, c, h, w, kh, kw, padding, stride)


def batch_norm(x, scale, bias, y, mean, invstd, eps):
    CALLS[0] += 1
    n, c, h, w = x.shape
    _rt().tsb_cpu_batchnorm(_p(x), _p(scale), _p(bias), _p(y), _p(mean), _p(invstd), n, c, h * w,
                                      c_float(eps))


def softmax_crossentropy(logits, labels, loss, dx=None):
    CALLS[0] += 1
    r, c = logits.shape
    _rt().tsb_cpu_softmax_ce(_p(logits), _p(labels), _p(loss), _p(dx) if dx is not None else None,
                                       c_int64(r), c_int64(c))


def optimizer_update(kind, p, g, s1, s2, hyper):
    CALLS[0] += 1
    h = (c_float * 8)(*(list(hyper) + [0.0] * (8 - len(hyper))))
    _rt().tsb_cpu_optimizer(kind, _p(p), _p(g), _p(s1) if s1 is not None else None,
                                      _p(s2) if s2 is not None else None, c_int64(p.size), h)


def conv2d_grad_data(dy, w, dx, padding=0, padding2=None, stride=1):
    CALLS[0] += 1
    n, c, h, wd = dx.shape
    o, _, kh, kw = w.shape
    pw = padding if padding2 is None else padding2
    _rt().tsb_cpu_conv2d_dgrad(_p(dy), _p(w), _p(dx), n, c, h, wd, o, kh, kw, dy.shape[2], dy.shape[3],
                                         padding, pw, stride)


def conv2d_grad_filter(x, dy, dw, padding=0, padding2=None, stride=1):
    CALLS[0] += 1
    n, c, h, wd = x.shape
    o, _, kh, kw = dw.shape
    pw = padding if padding2 is None else padding2
    _rt().tsb_cpu_conv2d_wgrad(_p(x), _p(dy), _p(dw), n, c, h, wd, o, kh, kw, dy.shape[2], dy.shape[3],
                                         padding, pw, stride)


def pool2d_grad(kind, x, dy, dx, kh, kw, padding, stride):
    CALLS[0] += 1
    n, c, h, w = dx.shape
    _rt().tsb_cpu_pool2d_grad(kind, _p(x) if x is not None else None, _p(dy), _p(dx), n, c, h, w, kh, kw,
                                        dy.shape[2], dy.shape[3], padding, stride)


def batch_norm_grad(dy, x, scale, bias, mean, invstd, dx, dscale, dbias, relu=False):
    CALLS[0] += 1
    n, c, h, w = x.shape
    _rt().tsb_cpu_batchnorm_grad(_p(dy), _p(x), _p(scale), _p(bias) if bias is not None else None, _p(mean),
                                           _p(invstd), _p(dx), _p(dscale), _p(dbias), n, c, h * w, int(relu))


def softmax(x, y):
    CALLS[0] += 1
    _rt().tsb_cpu_softmax(_p(x), _p(y), c_int64(x.size // x.shape[-1]), c_int64(x.shape[-1]))


def softmax_grad(y, dy, dx):
    CALLS[0] += 1
    _rt().tsb_cpu_softmax_grad(_p(y), _p(dy), _p(dx), c_int64(y.size // y.shape[-1]), c_int64(y.shape[-1]))


def reduce_sum_axis_zero(x, y):
    CALLS[0] += 1
    _rt().tsb_cpu_reduce_sum_axis0(_p(x), _p(y), c_int64(x.shape[0]), c_int64(x.size // x.shape[0]))


def broadcast_rows(x, y):
    """y[rows, ...] = x[...] for every leading index."""
    CALLS[0] += 1
    _rt().tsb_cpu_broadcast_rows(_p(x), _p(y), c_int64(y.size // x.size), c_int64(x.size))


def transpose(x, y, perm):
    CALLS[0] += 1
    nd = x.ndim
    _rt().tsb_cpu_transpose(_p(x), _p(y), nd, (c_int64 * nd)(*x.shape), (c_int * nd)(*perm))


def copy_block(x, y, outer, xcols, ycols, yoff, grad=False):
    """y[outer, yoff : yoff + xcols] <- x[outer, xcols] (or x <- that block of y when ``grad``)."""
    CALLS[0] += 1
    _rt().tsb_cpu_copy_block(_p(x), _p(y), c_int64(outer), c_int64(xcols), c_int64(ycols), c_int64(yoff),
                                       int(grad))


def pad2d(x, y, pads_h, pads_w, value=0.0, grad=False):
    """Constant padding of the two trailing axes (``grad``: x <- interior of y)."""
    CALLS[0] += 1
    h, w = x.shape[-2], x.shape[-1]
    _rt().tsb_cpu_pad2d(_p(x), _p(y), c_int64(x.size // (h * w)), h, w, pads_h[0], pads_h[1], pads_w[0],
                                  pads_w[1], c_float(value), int(grad))


def array_set(y, value):
    CALLS[0] += 1
    _rt().tsb_cpu_array_set(_p(y), c_int64(y.size), c_float(value))


def dropout(x, y, keep_prob, seed, offset=0):
    CALLS[0] += 1
    from ctypes import c_uint64
    _rt().tsb_cpu_dropout(_p(x), _p(y), c_int64(x.size), c_float(keep_prob), c_uint64(seed), c_int64(offset))


def softmax_crossentropy_grad(logits, labels, g, dx):
    CALLS[0] += 1
    r, c = logits.shape
    _rt().tsb_cpu_softmax_ce_grad(_p(logits), _p(labels), _p(g), _p(dx), c_int64(r), c_int64(c))
