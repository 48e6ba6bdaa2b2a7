"""Python entry points of the host operator library (role of the reference's
``python/athena/cpu_links/dnnl_op.py:8-274``): one thin function per C entry of
``csrc/runtime/cpu_ops.cc`` operating on contiguous fp32 NumPy arrays."""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p

import numpy as np

from . import _base


def _p(a):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return c_void_p(a.ctypes.data)


def matrix_multiply(a, b, c, trans_a=False, trans_b=False):
    m, n = c.shape
    k = a.shape[0] if trans_a else a.shape[1]
    _base.runtime().tsb_cpu_matmul(_p(a), _p(b), _p(c), m, n, k, int(trans_a), int(trans_b))


def binary(op, a, b, y):
    _base.runtime().tsb_cpu_binary(c_int(op), _p(a), _p(b), _p(y), c_int64(y.size))


def unary(op, x, y, alpha=0.0):
    _base.runtime().tsb_cpu_unary(c_int(op), _p(x), _p(y), c_int64(y.size), c_float(alpha))


def conv2d(x, w, y, padding=0, padding2=None, stride=1):
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    pw = padding if padding2 is None else padding2
    _base.runtime().tsb_cpu_conv2d(_p(x), _p(w), _p(y), n, c, h, wd, o, kh, kw, padding, pw, stride)


def pool2d(kind, x, y, kh, kw, padding, stride):
    n, c, h, w = x.shape
    _base.runtime().tsb_cpu_pool2d(kind, _p(x), _p(y), n, c, h, w, kh, kw, padding, stride)


def batch_norm(x, scale, bias, y, mean, invstd, eps):
    n, c, h, w = x.shape
    _base.runtime().tsb_cpu_batchnorm(_p(x), _p(scale), _p(bias), _p(y), _p(mean), _p(invstd), n, c, h * w,
                                      c_float(eps))


def softmax_crossentropy(logits, labels, loss, dx=None):
    r, c = logits.shape
    _base.runtime().tsb_cpu_softmax_ce(_p(logits), _p(labels), _p(loss), _p(dx) if dx is not None else None,
                                       c_int64(r), c_int64(c))


def optimizer_update(kind, p, g, s1, s2, hyper):
    h = (c_float * 8)(*(list(hyper) + [0.0] * (8 - len(hyper))))
    _base.runtime().tsb_cpu_optimizer(kind, _p(p), _p(g), _p(s1) if s1 is not None else None,
                                      _p(s2) if s2 is not None else None, c_int64(p.size), h)
