"""Softmax and softmax cross-entropy.

Capability parity: ``gpu_ops/Softmax.py:6-60`` and
``gpu_ops/SoftmaxCrossEntropy.py:39-118``.  The reference kernels run
``<<<1,1024>>>`` with one thread per row and a serial mean
(``src/ops/Softmax.cu:3-22``, ``SoftmaxCrossEntropy.cu:5-104``); here each row is
reduced by one warp (or one CTA for wide rows) across all SMs and the mean is a
deterministic two-stage reduction.
"""
from __future__ import annotations

import numpy as np

from ..graph import Op
from . import _gpu as G


def softmax_func(y):
    b = y - np.max(y, axis=-1, keepdims=True)
    e = np.exp(b)
    return e / np.sum(e, axis=-1, keepdims=True)


class SoftmaxOp(Op):
    name = "Softmax"

    def __call__(self, x):
        return Op.__call__(self, x)

    def np_compute(self, node, iv):
        return softmax_func(iv[0]).astype(np.float32)

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], out):
            return False
        cpu_links.softmax(iv[0], out)
        return True

    def gpu_compute(self, node, iv, out, stream):
        G.softmax(iv[0], out, stream)

    def gradient(self, node, g):
        # the reference leaves this undefined (src/ops/Softmax.cu has no backward kernel)
        return [softmax_gradient_op(node, g)]

    def infer_shape(self, node, s):
        return tuple(s[0])

    def flops(self, node, s, out):
        return 5.0 * np.prod(out)


class SoftmaxGradientOp(Op):
    """``dx = y * (dy - sum(dy * y, axis=-1, keepdims=True))`` in one kernel (y and dy read once)."""
    name = "SoftmaxGradient"

    def __call__(self, y, dy):
        return Op.__call__(self, y, dy)

    def np_compute(self, node, iv):
        y, dy = iv
        return (y * (dy - np.sum(dy * y, axis=-1, keepdims=True))).astype(np.float32)

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], iv[1], out):
            return False
        cpu_links.softmax_grad(iv[0], iv[1], out)
        return True

    def gpu_compute(self, node, iv, out, stream):
        G.softmax_grad(iv[0], iv[1], out, stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        assert tuple(s[0]) == tuple(s[1])
        return tuple(s[0])

    def flops(self, node, s, out):
        return 4.0 * np.prod(out)


class MaskedSoftmaxOp(Op):
    """Attention soft-max in one kernel: ``softmax(scale * scores + mask)`` over the last axis of
    ``scores [N, H, Tq, Tk]``.  ``key_tokens [N, Tk]`` (optional second input): keys whose token id is 0 are
    padding and get -1e9 added; ``causal``: keys behind the query (j > q) are replaced by -1e9.  Equals the chain
    the reference's example builds from separate operators (``examples/transformer.py:139-158``: scale, padding
    mask through a broadcast add, causal ``where``, soft-max), without their passes over the score tensor."""
    name = "MaskedSoftmax"

    def __call__(self, scores, key_tokens=None, scale=1.0, causal=False):
        ins = [scores] + ([key_tokens] if key_tokens is not None else [])
        return Op.__call__(self, *ins, scale=float(scale), causal=bool(causal))

    def np_compute(self, node, iv):
        x = iv[0].astype(np.float32) * np.float32(node.attrs["scale"])
        if len(iv) > 1:
            pad = (iv[1] == 0).astype(np.float32) * np.float32(-1e9)
            x = x + pad.reshape(pad.shape[0], 1, 1, pad.shape[-1])
        if node.attrs["causal"]:
            tq, tk = x.shape[-2], x.shape[-1]
            future = np.arange(tk)[None, :] > np.arange(tq)[:, None]
            x = np.where(future, np.float32(-1e9), x)
        return softmax_func(x).astype(np.float32)

    def gpu_compute(self, node, iv, out, stream):
        x = iv[0]
        assert x.is_contiguous() and out.is_contiguous() and len(x.shape) == 4
        key = iv[1] if len(iv) > 1 else None
        G.masked_softmax(x, key, out, node.attrs["scale"], node.attrs["causal"], stream)

    def gradient(self, node, g):
        grads = [masked_softmax_gradient_op(node, g, node.attrs["scale"])]
        if len(node.inputs) > 1:
            from .misc import zeroslike_op
            grads.append(zeroslike_op(node.inputs[1]))
        return grads

    def infer_shape(self, node, s):
        assert len(s[0]) == 4, "scores are [N, H, Tq, Tk]"
        if len(s) > 1:
            assert tuple(s[1]) == (s[0][0], s[0][3]), "key tokens are [N, Tk]"
        return tuple(s[0])

    def flops(self, node, s, out):
        return 7.0 * np.prod(out)


class MaskedSoftmaxGradientOp(Op):
    """``dx = scale * y * (dy - sum(dy * y, axis=-1, keepdims=True))`` (masked positions have y = 0)."""
    name = "MaskedSoftmaxGradient"

    def __call__(self, y, dy, scale=1.0):
        return Op.__call__(self, y, dy, scale=float(scale))

    def np_compute(self, node, iv):
        y, dy = iv
        return (np.float32(node.attrs["scale"]) * y * (dy - np.sum(dy * y, axis=-1, keepdims=True))).astype(np.float32)

    def gpu_compute(self, node, iv, out, stream):
        G.scaled_softmax_grad(iv[0], iv[1], out, node.attrs["scale"], stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        assert tuple(s[0]) == tuple(s[1])
        return tuple(s[0])

    def flops(self, node, s, out):
        return 5.0 * np.prod(out)


class SoftmaxCrossEntropyOp(Op):
    """``mean_rows(-sum(labels * log softmax(logits)))`` -> shape (1,)."""
    name = "SoftmaxCrossEntropy"

    def __call__(self, logits, labels):
        return Op.__call__(self, logits, labels)

    def np_compute(self, node, iv):
        y, y_ = iv
        b = y - np.max(y, axis=1, keepdims=True)
        logsm = b - np.log(np.sum(np.exp(b), axis=1, keepdims=True))
        return np.mean(-np.sum(y_ * logsm, axis=1), keepdims=True).astype(np.float32)

    def gpu_compute(self, node, iv, out, stream):
        G.softmax_ce(iv[0], iv[1], out, stream)

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], iv[1], out):
            return False
        cpu_links.softmax_crossentropy(iv[0], iv[1], out)
        return True

    def gradient(self, node, g):
        from .misc import zeroslike_op
        return [softmaxcrossentropy_gradient_op(node.inputs[0], node.inputs[1], g),
                zeroslike_op(node.inputs[1])]

    def infer_shape(self, node, s):
        assert tuple(s[0]) == tuple(s[1]), "logits %s and labels %s differ" % (s[0], s[1])
        return (1,)

    def flops(self, node, s, out):
        return 6.0 * np.prod(s[0])


class SoftmaxCrossEntropyGradientOp(Op):
    """``(softmax(logits) - labels) * g / rows``."""
    name = "SoftmaxCrossEntropyGradient"

    def __call__(self, logits, labels, g):
        return Op.__call__(self, logits, labels, g)

    def np_compute(self, node, iv):
        y, y_, g = iv
        return ((softmax_func(y) - y_) * g.reshape(-1)[0] / y.shape[0]).astype(np.float32)

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], iv[1], iv[2], out) or iv[0].ndim != 2 or iv[2].size != 1:
            return False
        cpu_links.softmax_crossentropy_grad(iv[0], iv[1], iv[2], out)
        return True

    def gpu_compute(self, node, iv, out, stream):
        G.softmax_ce_grad(iv[0], iv[1], iv[2], out, stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(s[0])

    def flops(self, node, s, out):
        return 6.0 * np.prod(out)


_sm, _ce, _ceg = SoftmaxOp(), SoftmaxCrossEntropyOp(), SoftmaxCrossEntropyGradientOp()
_smg = SoftmaxGradientOp()


def softmax_op(node):
    return _sm(node)


def softmax_gradient_op(node_y, node_dy):
    return _smg(node_y, node_dy)


_msm, _msmg = MaskedSoftmaxOp(), MaskedSoftmaxGradientOp()


def masked_softmax_op(scores, key_tokens=None, scale=1.0, causal=False):
    return _msm(scores, key_tokens, scale, causal)


def masked_softmax_gradient_op(node_y, node_dy, scale=1.0):
    return _msmg(node_y, node_dy, scale)


def softmaxcrossentropy_op(node_A, node_B):
    return _ce(node_A, node_B)


def softmaxcrossentropy_gradient_op(node_A, node_B, node_C):
    return _ceg(node_A, node_B, node_C)
