"""2-D convolution (NCHW x OIHW cross-correlation), its two gradients and the
per-channel bias helpers.

Capability parity: ``gpu_ops/Conv2d.py:100-138`` (forward), ``:227-266`` (data
gradient), ``:367-405`` (filter gradient), ``Conv2dBroadcast.py``,
``Conv2dReduceSum.py``; the reference computes on the GPU through cuDNN
(``src/ops/CudnnConv2d.cu:127-602``).

GPU path: implicit GEMM on the 5th-generation tensor cores
(``csrc/kernels/conv_tcgen05.cu``) — both operands arrive by TMA (the activation
patches through an im2col-mode tensor map that does padding, stride and image wrap
in the copy unit; channel counts that are no multiple of 32 fall back to ``cp.async``
gather warps), ``tcgen05.mma.kind::tf32`` accumulates in TMEM, CTA pairs
(``cta_group::2``) for 256-column tiles, output tiles leave by TMA store.  Operands are
channels-last.  The NumPy path (patch view + einsum) is the oracle; on a CPU context
the forward runs on the native host kernel (``cpu_links.conv2d``).
"""
from __future__ import annotations

import numpy as np

from ..graph import Op
from .. import ndarray
from . import _gpu as G


def out_hw(h, w, kh, kw, ph, pw, stride):
    return (h + 2 * ph - kh) // stride + 1, (w + 2 * pw - kw) // stride + 1


def _patches(x, kh, kw, ph, pw, stride):
    """[N, C, KH, KW, OH, OW] strided view of the zero-padded input."""
    n, c, h, w = x.shape
    xp = np.pad(x, ((0, 0), (0, 0), (ph, ph), (pw, pw)))
    oh, ow = out_hw(h, w, kh, kw, ph, pw, stride)
    s = xp.strides
    return np.lib.stride_tricks.as_strided(
        xp, (n, c, kh, kw, oh, ow), (s[0], s[1], s[2], s[3], s[2] * stride, s[3] * stride), writeable=False)


def np_conv2d(x, f, ph, pw, stride):
    o, c, kh, kw = f.shape
    p = _patches(x, kh, kw, ph, pw, stride)
    return np.einsum("nckluv,ockl->nouv", p, f, optimize=True).astype(np.float32)


def np_conv2d_grad_filter(x, gy, fshape, ph, pw, stride):
    o, c, kh, kw = fshape
    p = _patches(x, kh, kw, ph, pw, stride)
    return np.einsum("nckluv,nouv->ockl", p, gy, optimize=True).astype(np.float32)


def np_conv2d_grad_data(f, gy, xshape, ph, pw, stride):
    n, c, h, w = xshape
    o, _, kh, kw = f.shape
    _, _, oh, ow = gy.shape
    dxp = np.zeros((n, c, h + 2 * ph, w + 2 * pw), dtype=np.float32)
    for i in range(kh):
        for j in range(kw):
            contrib = np.einsum("nouv,oc->ncuv", gy, f[:, :, i, j], optimize=True)
            dxp[:, :, i:i + stride * oh:stride, j:j + stride * ow:stride] += contrib
    return dxp[:, :, ph:ph + h, pw:pw + w]


def _pads(node):
    ph = node.attrs["padding"]
    pw = node.attrs["padding2"]
    return ph, (ph if pw is None else pw)


class Conv2dOp(Op):
    name = "Conv2d"

    def __call__(self, x, f, padding=0, padding2=None, stride=1, For_ResNet=False):
        return Op.__call__(self, x, f, padding=padding, padding2=padding2, stride=stride,
                           For_ResNet=For_ResNet)

    def np_compute(self, node, iv):
        ph, pw = _pads(node)
        return np_conv2d(iv[0], iv[1], ph, pw, node.attrs["stride"])

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], iv[1], out):
            return False
        ph, pw = _pads(node)
        cpu_links.conv2d(iv[0], iv[1], out, ph, pw, node.attrs["stride"])
        return True

    def gpu_compute(self, node, iv, out, stream):
        ph, pw = _pads(node)
        bn = node.attrs.get("bn_consumer")
        if bn is not None:
            # a batch norm reads this output: take its column statistics in the epilogue
            st = bn.state
            o = out.shape[1]
            part = st.get("conv_part")
            if part is None or part.shape != (2 * G.CONV_STAT_MAX_CHUNKS * o,):
                part = st["conv_part"] = ndarray.empty((2 * G.CONV_STAT_MAX_CHUNKS * o,), out.ctx, use_pool=False)
            st["conv_chunks"] = G.conv2d_fwd_stats(iv[0], iv[1], out, ph, pw, node.attrs["stride"], part, stream)
            st["conv_rows"] = out.shape[0] * out.shape[2] * out.shape[3]
            return
        G.conv2d(0, iv[0], iv[1], out, ph, pw, node.attrs["stride"], stream)

    def gradient(self, node, g):
        x, f = node.inputs
        a = node.attrs
        return [conv2d_gradient_of_data_op(f, g, a["padding"], a["padding2"], a["stride"], a["For_ResNet"],
                                           like=x),
                conv2d_gradient_of_filter_op(x, g, a["padding"], a["padding2"], a["stride"], like=f)]

    def infer_shape(self, node, s):
        n, c, h, w = s[0]
        o, c2, kh, kw = s[1]
        assert c == c2, "conv2d: input has %d channels, filter expects %d" % (c, c2)
        ph, pw = _pads(node)
        oh, ow = out_hw(h, w, kh, kw, ph, pw, node.attrs["stride"])
        return (n, o, oh, ow)

    def flops(self, node, s, out):
        """Effective work for the cost model: thin reductions (few input channels)
        run below the tensor-core rate, so they are charged proportionally more."""
        o, c, kh, kw = s[1]
        k = c * kh * kw
        eff = min(1.0, (k / 1536.0) ** 0.5) * min(1.0, (o / 256.0) ** 0.5)
        return 2.0 * out[0] * out[2] * out[3] * o * c * kh * kw / max(eff, 0.05)

    def workspace_bytes(self, node, s, out):
        return 0


class Conv2dGradDataOp(Op):
    """dX.  The shape is the one inferred for the forward input (``like``, kept as
    an attribute, not a data dependency), which also covers the stride-2
    ambiguity the reference patches with its ``For_ResNet`` +1
    (``Conv2d.py:263-265``)."""
    name = "Conv2dGradData"

    def __call__(self, f, g, padding=0, padding2=None, stride=1, For_ResNet=False, like=None):
        return Op.__call__(self, f, g, padding=padding, padding2=padding2, stride=stride,
                           For_ResNet=For_ResNet, like=like)

    def _xshape(self, node, fs, gs):
        like = node.attrs["like"]
        if like is not None and getattr(like, "inferred_shape", None) is not None:
            return (gs[0],) + tuple(like.inferred_shape[1:])      # batch from the gradient (may be a piece)
        ph, pw = _pads(node)
        st = node.attrs["stride"]
        o, c, kh, kw = fs
        n, _, oh, ow = gs
        h = (oh - 1) * st + kh - 2 * ph
        w = (ow - 1) * st + kw - 2 * pw
        if node.attrs["For_ResNet"] and st == 2:
            h, w = h + 1, w + 1
        return (n, c, h, w)

    def np_compute(self, node, iv):
        ph, pw = _pads(node)
        xs = self._xshape(node, iv[0].shape, iv[1].shape)
        return np_conv2d_grad_data(iv[0], iv[1], xs, ph, pw, node.attrs["stride"])

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], iv[1], out):
            return False
        ph, pw = _pads(node)
        cpu_links.conv2d_grad_data(iv[1], iv[0], out, ph, pw, node.attrs["stride"])
        return True

    def gpu_compute(self, node, iv, out, stream):
        ph, pw = _pads(node)
        G.conv2d(1, out, iv[0], iv[1], ph, pw, node.attrs["stride"], stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return self._xshape(node, s[0], s[1])

    def flops(self, node, s, out):
        o, c, kh, kw = s[0]
        return 2.0 * s[1][0] * s[1][2] * s[1][3] * o * c * kh * kw


class Conv2dGradFilterOp(Op):
    name = "Conv2dGradFilter"

    def __call__(self, x, g, padding=0, padding2=None, stride=1, like=None, kernel=None):
        return Op.__call__(self, x, g, padding=padding, padding2=padding2, stride=stride,
                           like=like, kernel=kernel)

    def _fshape(self, node, xs, gs):
        like = node.attrs["like"]
        if like is not None and getattr(like, "inferred_shape", None) is not None:
            return tuple(like.inferred_shape)
        if node.attrs["kernel"] is not None:
            kh, kw = node.attrs["kernel"]
        else:
            ph, pw = _pads(node)
            st = node.attrs["stride"]
            kh = xs[2] + 2 * ph - (gs[2] - 1) * st
            kw = xs[3] + 2 * pw - (gs[3] - 1) * st
        return (gs[1], xs[1], kh, kw)

    def np_compute(self, node, iv):
        ph, pw = _pads(node)
        fs = self._fshape(node, iv[0].shape, iv[1].shape)
        return np_conv2d_grad_filter(iv[0], iv[1], fs, ph, pw, node.attrs["stride"])

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], iv[1], out):
            return False
        ph, pw = _pads(node)
        cpu_links.conv2d_grad_filter(iv[0], iv[1], out, ph, pw, node.attrs["stride"])
        return True

    def gpu_compute(self, node, iv, out, stream):
        ph, pw = _pads(node)
        G.conv2d(2, iv[0], out, iv[1], ph, pw, node.attrs["stride"], stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return self._fshape(node, s[0], s[1])

    def flops(self, node, s, out):
        return 2.0 * s[1][0] * s[1][2] * s[1][3] * out[0] * out[1] * out[2] * out[3]

    def workspace_bytes(self, node, s, out):
        # split-K partial sums live in a library-owned buffer outside the activation pool
        return 0


class Conv2dBroadcastToOp(Op):
    """bias (C,) -> (N, C, H, W) shaped like the second input."""
    name, cheap = "Conv2dBroadcastTo", True

    def __call__(self, bias, like):
        return Op.__call__(self, bias, like)

    def np_compute(self, node, iv):
        return np.broadcast_to(iv[0].reshape(1, -1, 1, 1), iv[1].shape).astype(np.float32)

    def gpu_compute(self, node, iv, out, stream):
        b = iv[0]
        G.copy_raw(b.ptr, [0, b.strides[-1], 0, 0], out.ptr, out.strides, out.shape, stream)

    def gradient(self, node, g):
        return [conv2d_reducesum_op(g), None]

    def infer_shape(self, node, s):
        return tuple(s[1])


class Conv2dReduceSumOp(Op):
    """(N, C, H, W) -> (C,) sum over N, H, W."""
    name = "Conv2dReduceSum"

    def __call__(self, x):
        return Op.__call__(self, x)

    def np_compute(self, node, iv):
        return iv[0].sum(axis=(0, 2, 3))

    def gpu_compute(self, node, iv, out, stream):
        x = iv[0]
        G.reduce_sum(x.ptr, list(x.shape), list(x.strides), [0, 2, 3], out, stream)

    def gradient(self, node, g):
        return [conv2d_broadcastto_op(g, node.inputs[0])]

    def infer_shape(self, node, s):
        return (s[0][1],)


_conv, _dgrad, _wgrad, _bcast, _rsum = (Conv2dOp(), Conv2dGradDataOp(), Conv2dGradFilterOp(),
                                        Conv2dBroadcastToOp(), Conv2dReduceSumOp())


def conv2d_op(node_A, node_B, padding=0, padding2=None, stride=1, For_ResNet=False):
    return _conv(node_A, node_B, padding, padding2, stride, For_ResNet)


def conv2d_gradient_of_data_op(node_A, node_B, padding=0, padding2=None, stride=1, For_ResNet=False,
                               like=None):
    """``node_A`` = filter, ``node_B`` = output gradient."""
    return _dgrad(node_A, node_B, padding, padding2, stride, For_ResNet, like)


def conv2d_gradient_of_filter_op(input_X, gradient_Y, padding=0, padding2=None, stride=1, like=None,
                                 kernel=None):
    return _wgrad(input_X, gradient_Y, padding, padding2, stride, like, kernel)


def conv2d_broadcastto_op(node_A, node_B):
    return _bcast(node_A, node_B)


def conv2d_reducesum_op(node_A):
    return _rsum(node_A)
