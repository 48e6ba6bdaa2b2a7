"""Inception-v4 (299x299, 1000 classes): stem, 4 x Inception-A, Reduction-A,
7 x Inception-B, Reduction-B, 3 x Inception-C, global average pool, dropout, FC —
the network of the reference's ``examples/imagenet_inceptionv4.py:84-262``, with
its asymmetric 1x7 / 7x1 / 1x3 / 3x1 convolutions (``padding`` = H pad,
``padding2`` = W pad)."""
from __future__ import annotations

from .. import gpu_ops as ad
from .common import Params, Model


class _Net(object):
    def __init__(self, p, div):
        self.p, self.div, self.i = p, div, 0

    def c(self, n):
        return max(n // self.div // 4 * 4, 4)

    def conv(self, x, cin, cout, kh, kw, stride=1, ph=0, pw=0):
        self.i += 1
        name = "incep_conv%d" % self.i
        w = self.p.he(name + "_weight", (cout, cin, kh, kw), cin * kh * kw)
        s = self.p.get(name + "_bn_scale", (1, cout, 1, 1), const=1.0)
        b = self.p.get(name + "_bn_bias", (1, cout, 1, 1), const=0.0)
        x = ad.conv2d_op(x, w, padding=ph, padding2=pw, stride=stride)
        return ad.batch_normalization_relu_op(x, s, b)


def _cat(parts):
    out = parts[0]
    for q in parts[1:]:
        out = ad.concat_op(out, q, axis=1)
    return out


def inception_v4(num_classes=1000, image=299, width_div=1, seed=123, dropout_keep=0.8):
    p = Params(seed)
    n = _Net(p, width_div)
    c = n.c
    X, y_ = ad.Variable(name="X"), ad.Variable(name="y_")
    # ---- stem
    x = n.conv(X, 3, c(32), 3, 3, stride=2)
    x = n.conv(x, c(32), c(32), 3, 3)
    x = n.conv(x, c(32), c(64), 3, 3, ph=1, pw=1)
    a = ad.max_pool2d_op(x, 3, 3, 0, 2)
    b = n.conv(x, c(64), c(96), 3, 3, stride=2)
    x = _cat([a, b]); ch = c(64) + c(96)
    a = n.conv(n.conv(x, ch, c(64), 1, 1), c(64), c(96), 3, 3)
    b = n.conv(x, ch, c(64), 1, 1)
    b = n.conv(b, c(64), c(64), 7, 1, ph=3, pw=0)
    b = n.conv(b, c(64), c(64), 1, 7, ph=0, pw=3)
    b = n.conv(b, c(64), c(96), 3, 3)
    x = _cat([a, b]); ch = 2 * c(96)
    a = n.conv(x, ch, c(192), 3, 3, stride=2)
    b = ad.max_pool2d_op(x, 3, 3, 0, 2)
    x = _cat([a, b]); ch = c(192) + ch
    # ---- 4 x Inception-A
    for _ in range(4):
        b0 = n.conv(ad.avg_pool2d_op(x, 3, 3, 1, 1), ch, c(96), 1, 1)
        b1 = n.conv(x, ch, c(96), 1, 1)
        b2 = n.conv(n.conv(x, ch, c(64), 1, 1), c(64), c(96), 3, 3, ph=1, pw=1)
        b3 = n.conv(x, ch, c(64), 1, 1)
        b3 = n.conv(b3, c(64), c(96), 3, 3, ph=1, pw=1)
        b3 = n.conv(b3, c(96), c(96), 3, 3, ph=1, pw=1)
        x = _cat([b0, b1, b2, b3]); ch = 4 * c(96)
    # ---- Reduction-A
    b0 = ad.max_pool2d_op(x, 3, 3, 0, 2)
    b1 = n.conv(x, ch, c(384), 3, 3, stride=2)
    b2 = n.conv(x, ch, c(192), 1, 1)
    b2 = n.conv(b2, c(192), c(224), 3, 3, ph=1, pw=1)
    b2 = n.conv(b2, c(224), c(256), 3, 3, stride=2)
    x = _cat([b0, b1, b2]); ch = ch + c(384) + c(256)
    # ---- 7 x Inception-B
    for _ in range(7):
        b0 = n.conv(ad.avg_pool2d_op(x, 3, 3, 1, 1), ch, c(128), 1, 1)
        b1 = n.conv(x, ch, c(384), 1, 1)
        b2 = n.conv(x, ch, c(192), 1, 1)
        b2 = n.conv(b2, c(192), c(224), 1, 7, ph=0, pw=3)
        b2 = n.conv(b2, c(224), c(256), 7, 1, ph=3, pw=0)
        b3 = n.conv(x, ch, c(192), 1, 1)
        b3 = n.conv(b3, c(192), c(192), 1, 7, ph=0, pw=3)
        b3 = n.conv(b3, c(192), c(224), 7, 1, ph=3, pw=0)
        b3 = n.conv(b3, c(224), c(224), 1, 7, ph=0, pw=3)
        b3 = n.conv(b3, c(224), c(256), 7, 1, ph=3, pw=0)
        x = _cat([b0, b1, b2, b3]); ch = c(128) + c(384) + 2 * c(256)
    # ---- Reduction-B
    b0 = ad.max_pool2d_op(x, 3, 3, 0, 2)
    b1 = n.conv(n.conv(x, ch, c(192), 1, 1), c(192), c(192), 3, 3, stride=2)
    b2 = n.conv(x, ch, c(256), 1, 1)
    b2 = n.conv(b2, c(256), c(256), 1, 7, ph=0, pw=3)
    b2 = n.conv(b2, c(256), c(320), 7, 1, ph=3, pw=0)
    b2 = n.conv(b2, c(320), c(320), 3, 3, stride=2)
    x = _cat([b0, b1, b2]); ch = ch + c(192) + c(320)
    # ---- 3 x Inception-C
    for _ in range(3):
        b0 = n.conv(ad.avg_pool2d_op(x, 3, 3, 1, 1), ch, c(256), 1, 1)
        b1 = n.conv(x, ch, c(256), 1, 1)
        b2 = n.conv(x, ch, c(384), 1, 1)
        b2a = n.conv(b2, c(384), c(256), 1, 3, ph=0, pw=1)
        b2b = n.conv(b2, c(384), c(256), 3, 1, ph=1, pw=0)
        b3 = n.conv(x, ch, c(384), 1, 1)
        b3 = n.conv(b3, c(384), c(448), 1, 3, ph=0, pw=1)
        b3 = n.conv(b3, c(448), c(512), 3, 1, ph=1, pw=0)
        b3a = n.conv(b3, c(512), c(256), 3, 1, ph=1, pw=0)
        b3b = n.conv(b3, c(512), c(256), 1, 3, ph=0, pw=1)
        x = _cat([b0, b1, b2a, b2b, b3a, b3b]); ch = 6 * c(256)
    # spatial size after the stem and two reductions
    hw = image
    hw = (hw - 3) // 2 + 1; hw = hw - 2; hw = (hw - 3) // 2 + 1; hw = hw - 2; hw = (hw - 3) // 2 + 1
    hw = (hw - 3) // 2 + 1; hw = (hw - 3) // 2 + 1
    x = ad.avg_pool2d_op(x, hw, hw, 0, hw)
    x = ad.array_reshape_op(x, (-1, ch))
    x = ad.dropout_op(x, dropout_keep, seed=seed + 17)
    w = p.he("incep_fc_weight", (ch, num_classes), ch)
    y = ad.matmul_op(x, w)
    loss = ad.softmaxcrossentropy_op(y, y_)
    return Model("inception_v4", X, y_, loss, y, p, (3, image, image), num_classes)
