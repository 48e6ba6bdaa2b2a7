"""Python entry points of the host operator library (role of the reference's
``python/athena/cpu_links/dnnl_op.py:8-274``): one thin function per C entry of
``csrc/runtime/cpu_ops.cc`` operating on contiguous fp32 NumPy arrays.  Executors on a
CPU context (``ndarray.cpu``) call them through ``Op.cpu_compute`` for matrix products,
convolution, pooling, the element-wise family and the softmax cross-entropy; operators
without a native kernel, and ``ctx=None`` (the NumPy oracle), use NumPy."""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p

import numpy as np

from . import _base


def _p(a):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return c_void_p(a.ctypes.data)


#: native kernel calls made so far (tests check that a CPU-context run really goes through the library)
CALLS = [0]


def ok(*arrays):
    """The native kernels take C-contiguous fp32 NumPy arrays."""
    return all(isinstance(a, np.ndarray) and a.dtype == np.float32 and a.flags.c_contiguous for a in arrays)


#: operator name -> code of tsb_cpu_unary / tsb_cpu_binary
UNARY = {"Relu": 1, "Sigmoid": 2, "Tanh": 3, "Sqrt": 4, "Rsqrt": 5, "Opposite": 6, "AddConst": 7, "MulConst": 8,
         "DivConst": 9}
BINARY = {"Add": 0, "Mul": 1, "Div": 2}


def matrix_multiply(a, b, c, trans_a=False, trans_b=False):
    CALLS[0] += 1
    m, n = c.shape
    k = a.shape[0] if trans_a else a.shape[1]
    _base.runtime().tsb_cpu_matmul(_p(a), _p(b), _p(c), m, n, k, int(trans_a), int(trans_b))


def binary(op, a, b, y):
    CALLS[0] += 1
    _base.runtime().tsb_cpu_binary(c_int(op), _p(a), _p(b), _p(y), c_int64(y.size))


def unary(op, x, y, alpha=0.0):
    CALLS[0] += 1
    _base.runtime().tsb_cpu_unary(c_int(op), _p(x), _p(y), c_int64(y.size), c_float(alpha))


def conv2d(x, w, y, padding=0, padding2=None, stride=1):
    CALLS[0] += 1
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    pw = padding if padding2 is None else padding2
    _base.runtime().tsb_cpu_conv2d(_p(x), _p(w), _p(y), n, c, h, wd, o, kh, kw, padding, pw, stride)


def pool2d(kind, x, y, kh, kw, padding, stride):
    CALLS[0] += 1
    n, c, h, w = x.shape
    _base.runtime().tsb_cpu_pool2d(kind, _p(x), _p(y), n, c, h, w, kh, kw, padding, stride)


def batch_norm(x, scale, bias, y, mean, invstd, eps):
    CALLS[0] += 1
    n, c, h, w = x.shape
    _base.runtime().tsb_cpu_batchnorm(_p(x), _p(scale), _p(bias), _p(y), _p(mean), _p(invstd), n, c, h * w,
                                      c_float(eps))


def softmax_crossentropy(logits, labels, loss, dx=None):
    CALLS[0] += 1
    r, c = logits.shape
    _base.runtime().tsb_cpu_softmax_ce(_p(logits), _p(labels), _p(loss), _p(dx) if dx is not None else None,
                                       c_int64(r), c_int64(c))


def optimizer_update(kind, p, g, s1, s2, hyper):
    CALLS[0] += 1
    h = (c_float * 8)(*(list(hyper) + [0.0] * (8 - len(hyper))))
    _base.runtime().tsb_cpu_optimizer(kind, _p(p), _p(g), _p(s1) if s1 is not None else None,
                                      _p(s2) if s2 is not None else None, c_int64(p.size), h)
