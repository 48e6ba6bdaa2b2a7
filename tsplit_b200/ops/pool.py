"""Max / average 2-D pooling and their gradients.

Capability parity: ``gpu_ops/MaxPool.py:97-128,173-200`` and
``gpu_ops/AvgPool.py:78-113,193-224`` (cuDNN ``MAX_DETERMINISTIC`` /
``AVERAGE_COUNT_INCLUDE_PADDING`` in ``src/ops/CudnnMaxPool.cu``,
``CudnnAvgPool.cu``).  GPU path: channels-last kernels, one thread per
(pixel, 4-channel vector); the max gradient is a gather over the windows that
contain an input pixel (deterministic, no atomics, first maximum wins as in the
NumPy oracle).
"""
from __future__ import annotations

import numpy as np

from ..graph import Op
from . import _gpu as G


def _windows(xp, kh, kw, stride, oh, ow):
    s = xp.strides
    return np.lib.stride_tricks.as_strided(
        xp, xp.shape[:2] + (oh, ow, kh, kw), (s[0], s[1], s[2] * stride, s[3] * stride, s[2], s[3]),
        writeable=False)


def _out_hw(h, w, kh, kw, pad, stride):
    return (h + 2 * pad - kh) // stride + 1, (w + 2 * pad - kw) // stride + 1


def np_max_pool(x, kh, kw, pad, stride):
    n, c, h, w = x.shape
    oh, ow = _out_hw(h, w, kh, kw, pad, stride)
    xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad)), constant_values=-np.inf)
    return _windows(xp, kh, kw, stride, oh, ow).max(axis=(4, 5)).astype(np.float32)


def np_max_pool_grad(x, y, gy, kh, kw, pad, stride):
    """Gradient goes to the first (row-major) maximum of each window."""
    n, c, h, w = x.shape
    oh, ow = gy.shape[2:]
    xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad)), constant_values=-np.inf)
    win = _windows(xp, kh, kw, stride, oh, ow).reshape(n, c, oh, ow, kh * kw)
    arg = win.argmax(axis=4)
    dxp = np.zeros_like(xp, dtype=np.float32)
    ni, ci, oi, oj = np.indices((n, c, oh, ow))
    ii = oi * stride + arg // kw
    jj = oj * stride + arg % kw
    np.add.at(dxp, (ni, ci, ii, jj), gy)
    return dxp[:, :, pad:pad + h, pad:pad + w]


def np_avg_pool(x, kh, kw, pad, stride):
    n, c, h, w = x.shape
    oh, ow = _out_hw(h, w, kh, kw, pad, stride)
    xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    return (_windows(xp, kh, kw, stride, oh, ow).sum(axis=(4, 5)) / float(kh * kw)).astype(np.float32)


def np_avg_pool_grad(gy, xshape, kh, kw, pad, stride):
    n, c, h, w = xshape
    oh, ow = gy.shape[2:]
    dxp = np.zeros((n, c, h + 2 * pad, w + 2 * pad), dtype=np.float32)
    for i in range(kh):
        for j in range(kw):
            dxp[:, :, i:i + stride * oh:stride, j:j + stride * ow:stride] += gy / float(kh * kw)
    return dxp[:, :, pad:pad + h, pad:pad + w]


class _PoolOp(Op):
    kind = 0

    def __call__(self, x, kernel_H, kernel_W, padding, stride):
        return Op.__call__(self, x, kernel_H=kernel_H, kernel_W=kernel_W, padding=padding, stride=stride)

    def _a(self, node):
        a = node.attrs
        return a["kernel_H"], a["kernel_W"], a["padding"], a["stride"]

    def gpu_compute(self, node, iv, out, stream):
        G.pool(self.kind, iv[0], out, *self._a(node), stream=stream)

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], out):
            return False
        kh, kw, pad, st = self._a(node)
        cpu_links.pool2d(self.kind, iv[0], out, kh, kw, pad, st)
        return True

    def infer_shape(self, node, s):
        n, c, h, w = s[0]
        kh, kw, pad, st = self._a(node)
        oh, ow = _out_hw(h, w, kh, kw, pad, st)
        return (n, c, oh, ow)

    def flops(self, node, s, out):
        kh, kw, _, _ = self._a(node)
        return float(out[0] * out[1] * out[2] * out[3] * kh * kw)


class MaxPool2dOp(_PoolOp):
    name, kind = "MaxPool2d", 0

    def np_compute(self, node, iv):
        return np_max_pool(iv[0], *self._a(node))

    def gradient(self, node, g):
        return [max_pool2d_gradient_op(node, g, node.inputs[0], *self._a(node))]


class AvgPool2dOp(_PoolOp):
    name, kind = "AvgPool2d", 1

    def np_compute(self, node, iv):
        return np_avg_pool(iv[0], *self._a(node))

    def gradient(self, node, g):
        return [avg_pool2d_gradient_op(node, g, node.inputs[0], *self._a(node))]


class MaxPool2dGradientOp(Op):
    name = "MaxPool2dGradient"

    def __call__(self, y, gy, x, kernel_H, kernel_W, padding, stride):
        return Op.__call__(self, y, gy, x, kernel_H=kernel_H, kernel_W=kernel_W, padding=padding,
                           stride=stride)

    def np_compute(self, node, iv):
        a = node.attrs
        return np_max_pool_grad(iv[2], iv[0], iv[1], a["kernel_H"], a["kernel_W"], a["padding"], a["stride"])

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[1], iv[2], out):
            return False
        a = node.attrs
        cpu_links.pool2d_grad(0, iv[2], iv[1], out, a["kernel_H"], a["kernel_W"], a["padding"], a["stride"])
        return True

    def gpu_compute(self, node, iv, out, stream):
        a = node.attrs
        G.pool_grad(0, iv[2], iv[0], iv[1], out, a["kernel_H"], a["kernel_W"], a["padding"], a["stride"], stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(s[2])


class AvgPool2dGradientOp(Op):
    """Needs only the output gradient; the input shape comes from the forward
    input's inferred shape (attribute ``like``), so the activation is not kept
    alive for the backward pass."""
    name = "AvgPool2dGradient"

    def __call__(self, y, gy, x, kernel_H, kernel_W, padding, stride):
        return Op.__call__(self, gy, like=x, kernel_H=kernel_H, kernel_W=kernel_W, padding=padding,
                           stride=stride)

    def np_compute(self, node, iv):
        a = node.attrs
        xs = (iv[0].shape[0],) + tuple(a["like"].inferred_shape[1:])       # batch from the gradient (may be a piece)
        return np_avg_pool_grad(iv[0], xs, a["kernel_H"], a["kernel_W"],
                                a["padding"], a["stride"])

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], out):
            return False
        a = node.attrs
        cpu_links.pool2d_grad(1, None, iv[0], out, a["kernel_H"], a["kernel_W"], a["padding"], a["stride"])
        return True

    def gpu_compute(self, node, iv, out, stream):
        a = node.attrs
        G.pool_grad(1, None, None, iv[0], out, a["kernel_H"], a["kernel_W"], a["padding"], a["stride"], stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(node.attrs["like"].inferred_shape)


_maxp, _avgp, _maxg, _avgg = MaxPool2dOp(), AvgPool2dOp(), MaxPool2dGradientOp(), AvgPool2dGradientOp()


def max_pool2d_op(node_A, kernel_H, kernel_W, padding, stride):
    return _maxp(node_A, kernel_H, kernel_W, padding, stride)


def max_pool2d_gradient_op(node_out, node_out_gradient, node_in, kernel_H, kernel_W, padding, stride):
    return _maxg(node_out, node_out_gradient, node_in, kernel_H, kernel_W, padding, stride)


def avg_pool2d_op(node_A, kernel_H, kernel_W, padding, stride):
    return _avgp(node_A, kernel_H, kernel_W, padding, stride)


def avg_pool2d_gradient_op(node_out, node_out_gradient, node_in, kernel_H, kernel_W, padding, stride):
    return _avgg(node_out, node_out_gradient, node_in, kernel_H, kernel_W, padding, stride)
