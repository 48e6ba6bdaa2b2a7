"""VGG-16 / VGG-19 with batch-norm (13 or 16 conv3x3 + 3 FC, 1000 classes),
the architecture of the reference's ``examples/imagenet_vgg.py:24-98``."""
from __future__ import annotations

from .. import gpu_ops as ad
from .common import Params, Model

_CFG = {16: [2, 2, 3, 3, 3], 19: [2, 2, 4, 4, 4]}
_WIDTH = [64, 128, 256, 512, 512]


def conv_bn_relu(p, x, cin, cout, name):
    w = p.he(name + "_weight", (cout, cin, 3, 3), cin * 9)
    scale = p.get(name + "_bn_scale", (1, cout, 1, 1), const=1.0)
    bias = p.get(name + "_bn_bias", (1, cout, 1, 1), const=0.0)
    x = ad.conv2d_op(x, w, padding=1, stride=1)
    return ad.batch_normalization_relu_op(x, scale, bias)


def vgg(num_layers=16, num_classes=1000, image=224, width_div=1, fc_width=4096, seed=123):
    """``width_div`` / ``fc_width`` / ``image`` shrink the net for tests; the
    defaults are the real VGG."""
    assert num_layers in _CFG, "VGG model should have 16 or 19 layers!"
    p = Params(seed)
    X, y_ = ad.Variable(name="X"), ad.Variable(name="y_")
    x, cin, hw = X, 3, image
    for b, (reps, cout) in enumerate(zip(_CFG[num_layers], _WIDTH)):
        cout = max(cout // width_div, 4)
        for r in range(reps):
            x = conv_bn_relu(p, x, cin, cout, "vgg_block%d_layer%d" % (b + 1, r + 1))
            cin = cout
        x = ad.max_pool2d_op(x, kernel_H=2, kernel_W=2, padding=0, stride=2)
        hw //= 2
    feat = hw * hw * cin
    x = ad.array_reshape_op(x, (-1, feat))
    w1 = p.he("vgg_fc1_weight", (feat, fc_width), feat)
    w2 = p.he("vgg_fc2_weight", (fc_width, fc_width), fc_width)
    w3 = p.he("vgg_fc3_weight", (fc_width, num_classes), fc_width)
    x = ad.relu_op(ad.matmul_op(x, w1))
    x = ad.relu_op(ad.matmul_op(x, w2))
    y = ad.matmul_op(x, w3)
    loss = ad.softmaxcrossentropy_op(y, y_)
    return Model("vgg%d" % num_layers, X, y_, loss, y, p, (3, image, image), num_classes)
