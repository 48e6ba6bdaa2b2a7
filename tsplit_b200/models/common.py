"""Shared model-building helpers: variable registry with random initial values."""
from __future__ import annotations

import numpy as np

from .. import gpu_ops as ad


class Params(object):
    """Creates trainable variables with N(0, scale) (or constant) initial values
    and remembers them in creation order (the reference's examples keep two
    parallel global lists, ``examples/imagenet_vgg.py:8-22``)."""

    def __init__(self, seed=123, scale=0.1):
        self.rand = np.random.RandomState(seed)
        self.scale = scale
        self.variables = []

    def get(self, name, shape, scale=None, const=None):
        if const is not None:
            val = np.full(shape, const, dtype=np.float32)
        else:
            val = self.rand.normal(scale=self.scale if scale is None else scale, size=shape).astype(np.float32)
        v = ad.Variable(name=name, value=val)
        self.variables.append(v)
        return v

    def he(self, name, shape, fan_in):
        return self.get(name, shape, scale=float(np.sqrt(2.0 / fan_in)))

    def num_parameters(self):
        return int(sum(np.prod(v.tensor_value.shape) for v in self.variables))


class Model(object):
    """What every model builder returns."""

    def __init__(self, name, X, y_, loss, y, params, input_shape, num_classes):
        self.name, self.X, self.y_, self.loss, self.y = name, X, y_, loss, y
        self.params = params
        self.variables = params.variables
        self.input_shape = tuple(input_shape)     # per-sample shape
        self.num_classes = num_classes

    def synthetic_batch(self, batch, seed=0):
        r = np.random.RandomState(seed)
        x = r.standard_normal((batch,) + self.input_shape).astype(np.float32)
        y = np.eye(self.num_classes, dtype=np.float32)[r.randint(0, self.num_classes, batch)]
        return x, y
