"""ResNet-50 / 101 (bottleneck [3,4,6,3] / [3,4,23,3], BN, 1000 classes), the
architecture of the reference's ``examples/imagenet_resnet.py:45-121``."""
from __future__ import annotations

from .. import gpu_ops as ad
from .common import Params, Model

_BLOCKS = {50: [3, 4, 6, 3], 101: [3, 4, 23, 3], 26: [2, 2, 2, 2]}


def conv_bn(p, x, cin, cout, k, stride, pad, name, relu=True):
    w = p.he(name + "_weight", (cout, cin, k, k), cin * k * k)
    scale = p.get(name + "_bn_scale", (1, cout, 1, 1), const=1.0)
    bias = p.get(name + "_bn_bias", (1, cout, 1, 1), const=0.0)
    x = ad.conv2d_op(x, w, padding=pad, stride=stride)
    return ad.batch_normalization_relu_op(x, scale, bias) if relu else ad.batch_normalization_op(x, scale, bias)


def bottleneck(p, x, cin, mid, stride, name):
    cout = mid * 4
    y = conv_bn(p, x, cin, mid, 1, 1, 0, name + "_a")
    y = conv_bn(p, y, mid, mid, 3, stride, 1, name + "_b")
    y = conv_bn(p, y, mid, cout, 1, 1, 0, name + "_c", relu=False)
    if stride != 1 or cin != cout:
        x = conv_bn(p, x, cin, cout, 1, stride, 0, name + "_proj", relu=False)
    return ad.add_relu_op(x, y), cout


def resnet(num_layers=50, num_classes=1000, image=224, width_div=1, seed=123):
    p = Params(seed)
    X, y_ = ad.Variable(name="X"), ad.Variable(name="y_")
    base = max(64 // width_div, 4)
    x = conv_bn(p, X, 3, base, 7, 2, 3, "resnet_stem")
    x = ad.max_pool2d_op(x, kernel_H=3, kernel_W=3, padding=1, stride=2)
    cin, hw = base, image // 4
    for s, reps in enumerate(_BLOCKS[num_layers]):
        mid = base * (2 ** s)
        for r in range(reps):
            stride = 2 if (r == 0 and s > 0) else 1
            x, cin = bottleneck(p, x, cin, mid, stride, "resnet_s%d_b%d" % (s + 1, r + 1))
            if stride == 2:
                hw //= 2
    x = ad.avg_pool2d_op(x, kernel_H=hw, kernel_W=hw, padding=0, stride=hw)
    x = ad.array_reshape_op(x, (-1, cin))
    w = p.he("resnet_fc_weight", (cin, num_classes), cin)
    y = ad.matmul_op(x, w)
    loss = ad.softmaxcrossentropy_op(y, y_)
    return Model("resnet%d" % num_layers, X, y_, loss, y, p, (3, image, image), num_classes)
