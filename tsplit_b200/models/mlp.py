"""MLP 784-256-256-10 without bias (the plumbing config of the reference's
README, ``README.md:38-41``)."""
from __future__ import annotations

from .. import gpu_ops as ad
from .common import Params, Model


def mlp(sizes=(784, 256, 256, 10), seed=123):
    p = Params(seed)
    X, y_ = ad.Variable(name="X"), ad.Variable(name="y_")
    x = X
    for i in range(len(sizes) - 1):
        w = p.get("mlp_fc%d_weight" % (i + 1), (sizes[i], sizes[i + 1]), scale=0.1)
        x = ad.matmul_op(x, w)
        if i + 2 < len(sizes):
            x = ad.relu_op(x)
    loss = ad.softmaxcrossentropy_op(x, y_)
    return Model("mlp", X, y_, loss, x, p, (sizes[0],), sizes[-1])
