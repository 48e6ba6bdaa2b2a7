"""LSTM classifier over 28 steps of 28 features (MNIST rows), hidden 128 — the
model of the reference's ``examples/LSTM.py:22-86``: four gates from two matmuls
per step, sigmoid / tanh, final dense layer."""
from __future__ import annotations

import numpy as np

from .. import gpu_ops as ad
from .common import Params, Model


def lstm(steps=28, features=28, hidden=128, num_classes=10, seed=123):
    p = Params(seed)
    X, y_ = ad.Variable(name="X"), ad.Variable(name="y_")          # X: (N, steps*features)
    gates = {}
    for g in ("forget", "input", "output", "cell"):
        gates[g] = (p.get("lstm_%s_w" % g, (features, hidden)), p.get("lstm_%s_u" % g, (hidden, hidden)),
                    p.get("lstm_%s_b" % g, (hidden,), const=0.0))
    h = c = None
    for t in range(steps):
        x_t = ad.slice_op(X, (0, t * features), (-1, features))

        def gate(name, act):
            w, u, b = gates[name]
            z = ad.matmul_op(x_t, w)
            if h is not None:
                z = z + ad.matmul_op(h, u)
            z = z + ad.broadcasttoTF_op(b, z)
            return act(z)
        f, i, o = gate("forget", ad.sigmoid_op), gate("input", ad.sigmoid_op), gate("output", ad.sigmoid_op)
        g = gate("cell", ad.tanh_op)
        c = ad.mul_op(i, g) if c is None else ad.mul_op(f, c) + ad.mul_op(i, g)
        h = ad.mul_op(o, ad.tanh_op(c))
    w = p.get("lstm_dense_w", (hidden, num_classes))
    b = p.get("lstm_dense_b", (num_classes,), const=0.0)
    y = ad.matmul_op(h, w)
    y = y + ad.broadcasttoTF_op(b, y)
    loss = ad.softmaxcrossentropy_op(y, y_)
    return Model("lstm", X, y_, loss, y, p, (steps * features,), num_classes)
