"""Batch normalisation (spatial, training mode) and layer normalisation.

Capability parity: ``gpu_ops/BatchNorm.py:54-96`` (exported op) and
``gpu_ops/BatchNorm2.py:106-114`` (full three-gradient variant) over cuDNN
``cudnnBatchNormalizationForwardTraining/Backward`` (``src/ops/CudnnBn.cu``).

Deliberate deviations from the reference, which this build treats as defects:
scale and bias DO receive gradients (the exported reference op returns
``[dx, None, None]``), running mean/variance persist across steps (the
reference zeroes and frees them every call, ``CudnnBn.cu:77-88``), and the
NumPy gradient divides by N*H*W rather than by the channel count
(``BatchNorm.py:503-544``).  Defaults ``momentum=0.99, eps=0.01`` are kept.

GPU path (``csrc/kernels/norm.cu``): channels-last column statistics with a
two-stage deterministic reduction, then one fused normalise+scale+shift pass;
backward is one statistics pass plus one fused dx pass.
"""
from __future__ import annotations

import numpy as np

from ..graph import Op
from .. import ndarray
from . import _gpu as G


def np_bn_forward(x, scale, bias, eps):
    c = x.shape[1]
    mean = x.mean(axis=(0, 2, 3), dtype=np.float64)
    var = x.var(axis=(0, 2, 3), dtype=np.float64)
    invstd = 1.0 / np.sqrt(var + eps)
    xn = (x - mean.reshape(1, c, 1, 1)) * invstd.reshape(1, c, 1, 1)
    y = scale.reshape(1, c, 1, 1) * xn + bias.reshape(1, c, 1, 1)
    return y.astype(np.float32), mean.astype(np.float32), var.astype(np.float32), invstd.astype(np.float32)


def np_bn_backward(gy, x, scale, mean, invstd):
    c = x.shape[1]
    m = x.shape[0] * x.shape[2] * x.shape[3]
    xn = (x - mean.reshape(1, c, 1, 1)) * invstd.reshape(1, c, 1, 1)
    dscale = (gy * xn).sum(axis=(0, 2, 3), dtype=np.float64)
    dbias = gy.sum(axis=(0, 2, 3), dtype=np.float64)
    dx = (scale.reshape(1, c, 1, 1) * invstd.reshape(1, c, 1, 1)) * (
        gy - dbias.reshape(1, c, 1, 1) / m - xn * dscale.reshape(1, c, 1, 1) / m)
    return dx.astype(np.float32), dscale.astype(np.float32), dbias.astype(np.float32)


def _small(shape, ctx, value=None):
    """Per-node side buffer (statistics, parameter gradients): tiny, so it lives
    outside the capped activation pool."""
    a = ndarray.empty(shape, ctx, use_pool=False)
    if value is not None:
        a.t.fill_(value)
    return a


class BatchNormOp(Op):
    name = "BatchNorm"

    def __call__(self, x, scale, bias, momentum=0.99, eps=0.01):
        node = Op.__call__(self, x, scale, bias, momentum=momentum, eps=eps)
        node.state = {}
        if getattr(x.op, "name", None) == "Conv2d" and x.attrs.get("bn_consumer") is None:
            x.attrs["bn_consumer"] = node      # the convolution's epilogue then supplies the column statistics
        return node

    def _forward(self, node, iv, out, stream, relu):
        x, scale, bias = iv
        st = node.state
        c = x.shape[1]
        if "mean" not in st or st["mean"].shape != (c,):
            st["mean"], st["invstd"] = _small((c,), x.ctx), _small((c,), x.ctx)
            st["run_mean"], st["run_var"] = _small((c,), x.ctx, 0.0), _small((c,), x.ctx, 1.0)
        if st.get("rematerialise"):      # same step, statistics known: normalise only, leave running stats alone
            return G.bn_apply(x, scale, bias, out, st["mean"], st["invstd"], relu, stream)
        chunks = st.pop("conv_chunks", 0)
        if chunks and st.get("conv_rows") == x.shape[0] * x.shape[2] * x.shape[3]:
            return G.bn_forward_from_partials(st["conv_part"], chunks, x, scale, bias, out, st["mean"], st["invstd"],
                                              st["run_mean"], st["run_var"], node.attrs["momentum"],
                                              node.attrs["eps"], relu, stream)
        G.bn_forward(x, scale, bias, out, st["mean"], st["invstd"], st["run_mean"], st["run_var"],
                     node.attrs["momentum"], node.attrs["eps"], relu, stream)

    def np_compute(self, node, iv):
        x, scale, bias = iv
        y, mean, var, invstd = np_bn_forward(x, scale, bias, node.attrs["eps"])
        st = node.state
        mom = node.attrs["momentum"]
        st["np_mean"], st["np_invstd"] = mean, invstd
        st["np_run_mean"] = mom * st.get("np_run_mean", np.zeros_like(mean)) + (1 - mom) * mean
        st["np_run_var"] = mom * st.get("np_run_var", np.ones_like(var)) + (1 - mom) * var
        return y

    def cpu_compute(self, node, iv, out, relu=False):
        from .. import cpu_links
        x, scale, bias = iv
        if x.ndim != 4 or not cpu_links.ok(x, scale, bias, out):
            return False
        c = x.shape[1]
        mean, invstd = np.empty(c, np.float32), np.empty(c, np.float32)
        cpu_links.batch_norm(x, scale, bias, out, mean, invstd, node.attrs["eps"])
        if relu:
            cpu_links.unary(cpu_links.UNARY["Relu"], out, out)
        st, mom = node.state, node.attrs["momentum"]
        var = 1.0 / (invstd.astype(np.float64) ** 2) - node.attrs["eps"]
        st["np_mean"], st["np_invstd"] = mean, invstd
        st["np_run_mean"] = mom * st.get("np_run_mean", np.zeros_like(mean)) + (1 - mom) * mean
        st["np_run_var"] = mom * st.get("np_run_var", np.ones_like(mean)) + (1 - mom) * var.astype(np.float32)
        return True

    def gpu_compute(self, node, iv, out, stream):
        self._forward(node, iv, out, stream, False)

    def gradient(self, node, g):
        x, scale, bias = node.inputs
        bg = batch_normalization_gradient_op(g, x, scale, node.attrs["eps"], fwd=node)
        return [bg,
                batch_normalization_gradient_of_scale_op(bg, scale),
                batch_normalization_gradient_of_bias_op(bg, bias)]

    def infer_shape(self, node, s):
        return tuple(s[0])

    def flops(self, node, s, out):
        return 8.0 * np.prod(out)


class BatchNormReluOp(BatchNormOp):
    """``relu(batch_norm(x))`` in one pass over the data (the normalise / scale /
    shift kernel applies the ReLU before it stores), with a backward that masks
    the incoming gradient on the fly by the sign of the forward output, which it
    recomputes from ``x``, ``scale`` and ``bias`` (so the output itself is not an
    input of the backward node and is not read again).  Compared with the two-node
    form this removes one activation tensor and four memory passes per layer."""
    name = "BatchNormRelu"

    def np_compute(self, node, iv):
        return np.maximum(BatchNormOp.np_compute(self, node, iv), 0)

    def cpu_compute(self, node, iv, out):
        return BatchNormOp.cpu_compute(self, node, iv, out, relu=True)

    def gpu_compute(self, node, iv, out, stream):
        self._forward(node, iv, out, stream, True)

    def gradient(self, node, g):
        x, scale, bias = node.inputs
        bg = _bnrg(g, x, scale, bias, eps=node.attrs["eps"], fwd=node)
        return [bg, batch_normalization_gradient_of_scale_op(bg, scale),
                batch_normalization_gradient_of_bias_op(bg, bias)]


class BatchNormReluGradientOp(Op):
    name = "BatchNormReluGradient"

    def __call__(self, g, x, scale, bias, eps=0.01, fwd=None):
        node = Op.__call__(self, g, x, scale, bias, eps=eps, fwd=fwd)
        node.state = {}
        return node

    def np_compute(self, node, iv):
        g, x, scale, bias = iv
        fwd = node.attrs["fwd"]
        mean, invstd = fwd.state["np_mean"], fwd.state["np_invstd"]
        bc = (1, -1, 1, 1)
        y = (x - mean.reshape(bc)) * invstd.reshape(bc) * scale.reshape(bc) + bias.reshape(bc)
        dx, ds, db = np_bn_backward(g * (y > 0), x, scale, mean, invstd)
        node.state["np_dscale"], node.state["np_dbias"] = ds.reshape(scale.shape), db.reshape(scale.shape)
        return dx

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        g, x, scale, bias = iv
        fwd = node.attrs["fwd"]
        if x.ndim != 4 or fwd is None or "np_mean" not in fwd.state or not cpu_links.ok(g, x, scale, bias, out):
            return False
        ds, db = np.empty(scale.shape, np.float32), np.empty(scale.shape, np.float32)
        cpu_links.batch_norm_grad(g, x, scale, bias, np.ascontiguousarray(fwd.state["np_mean"], np.float32),
                                  np.ascontiguousarray(fwd.state["np_invstd"], np.float32), out, ds, db, relu=True)
        node.state["np_dscale"], node.state["np_dbias"] = ds, db
        return True

    def gpu_compute(self, node, iv, out, stream):
        g, x, scale, bias = iv
        fwd, st = node.attrs["fwd"], node.state
        if "dscale" not in st or st["dscale"].shape != tuple(scale.shape):
            st["dscale"], st["dbias"] = _small(scale.shape, x.ctx), _small(scale.shape, x.ctx)
        G.bn_relu_backward(g, x, scale, bias, fwd.state["mean"], fwd.state["invstd"], out, st["dscale"],
                           st["dbias"], stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(s[1])

    def flops(self, node, s, out):
        return 13.0 * np.prod(out)


class BatchNormGradientOp(Op):
    """Computes dx (its output) and keeps dscale / dbias in side buffers that the
    ``..._of_scale`` / ``..._of_bias`` nodes hand out."""
    name = "BatchNormGradient"

    def __call__(self, g, x, scale, eps, fwd=None):
        node = Op.__call__(self, g, x, scale, eps=eps, fwd=fwd)
        node.state = {}
        return node

    def _stats(self, node, x, scale_shape):
        fwd = node.attrs["fwd"]
        if fwd is not None and "np_mean" in fwd.state:
            return fwd.state["np_mean"], fwd.state["np_invstd"]
        mean = x.mean(axis=(0, 2, 3))
        return mean, 1.0 / np.sqrt(x.var(axis=(0, 2, 3)) + node.attrs["eps"])

    def np_compute(self, node, iv):
        g, x, scale = iv
        mean, invstd = self._stats(node, x, scale.shape)
        dx, ds, db = np_bn_backward(g, x, scale, mean, invstd)
        node.state["np_dscale"], node.state["np_dbias"] = ds.reshape(scale.shape), db.reshape(scale.shape)
        return dx

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        g, x, scale = iv
        fwd = node.attrs["fwd"]
        if x.ndim != 4 or fwd is None or "np_mean" not in fwd.state or not cpu_links.ok(g, x, scale, out):
            return False
        ds, db = np.empty(scale.shape, np.float32), np.empty(scale.shape, np.float32)
        cpu_links.batch_norm_grad(g, x, scale, None, np.ascontiguousarray(fwd.state["np_mean"], np.float32),
                                  np.ascontiguousarray(fwd.state["np_invstd"], np.float32), out, ds, db, relu=False)
        node.state["np_dscale"], node.state["np_dbias"] = ds, db
        return True

    def gpu_compute(self, node, iv, out, stream):
        g, x, scale = iv
        fwd = node.attrs["fwd"]
        st = node.state
        c = x.shape[1]
        if "dscale" not in st or st["dscale"].shape != tuple(scale.shape):
            st["dscale"], st["dbias"] = _small(scale.shape, x.ctx), _small(scale.shape, x.ctx)
        assert fwd is not None and "mean" in fwd.state, "batch-norm backward needs the forward statistics"
        G.bn_backward(g, x, scale, fwd.state["mean"], fwd.state["invstd"], out, st["dscale"], st["dbias"],
                      stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(s[1])

    def flops(self, node, s, out):
        return 12.0 * np.prod(out)


class _BnGradPick(Op):
    which = "dx"
    cheap = True

    def __call__(self, bn_grad, like):
        return Op.__call__(self, bn_grad, like)

    def gradient(self, node, g):
        raise NotImplementedError


class BatchNormGradDataOp(_BnGradPick):
    """Identity on the gradient node's output (kept for API parity); executors
    alias it to its input instead of copying."""
    name = "BatchNormGradData"
    alias_input = 0

    def np_compute(self, node, iv):
        return iv[0]

    def gpu_compute(self, node, iv, out, stream):
        if out is not iv[0] and out.ptr != iv[0].ptr:
            G.copy(iv[0], out, stream)

    def infer_shape(self, node, s):
        return tuple(s[0])


class BatchNormGradScaleOp(_BnGradPick):
    name, key = "BatchNormGradScale", "dscale"

    def np_compute(self, node, iv):
        return node.inputs[0].state["np_" + self.key]

    def gpu_compute(self, node, iv, out, stream):
        G.copy(node.inputs[0].state[self.key], out, stream)

    def infer_shape(self, node, s):
        return tuple(s[1])


class BatchNormGradBiasOp(BatchNormGradScaleOp):
    name, key = "BatchNormGradBias", "dbias"


# ---------------------------------------------------------------------------------
class LayerNormOp(Op):
    """Normalise over the last dimension; scale / bias of shape (D,).  Not in the
    reference op list (its transformer composes reductions); provided because
    the fused kernel replaces six memory passes with one."""
    name = "LayerNorm"

    def __call__(self, x, scale, bias, eps=1e-5):
        node = Op.__call__(self, x, scale, bias, eps=eps)
        node.state = {}
        return node

    def np_compute(self, node, iv):
        x, scale, bias = iv
        mean = x.mean(axis=-1, keepdims=True)
        invstd = 1.0 / np.sqrt(x.var(axis=-1, keepdims=True) + node.attrs["eps"])
        node.state["np_mean"], node.state["np_invstd"] = mean, invstd
        return ((x - mean) * invstd * scale + bias).astype(np.float32)

    def gpu_compute(self, node, iv, out, stream):
        x, scale, bias = iv
        rows = int(np.prod(x.shape[:-1]))
        st = node.state
        if "mean" not in st or st["mean"].shape != (rows,):
            st["mean"], st["invstd"] = _small((rows,), x.ctx), _small((rows,), x.ctx)
        G.layer_norm(x, scale, bias, out, st["mean"], st["invstd"], node.attrs["eps"], stream)

    def gradient(self, node, g):
        x, scale, bias = node.inputs
        lg = _lng(g, x, scale, fwd=node)
        return [lg, _lng_scale(lg, scale), _lng_bias(lg, bias)]

    def infer_shape(self, node, s):
        return tuple(s[0])


class LayerNormGradientOp(Op):
    name = "LayerNormGradient"

    def __call__(self, g, x, scale, fwd=None):
        node = Op.__call__(self, g, x, scale, fwd=fwd)
        node.state = {}
        return node

    def np_compute(self, node, iv):
        g, x, scale = iv
        fwd = node.attrs["fwd"]
        mean, invstd = fwd.state["np_mean"], fwd.state["np_invstd"]
        d = x.shape[-1]
        xn = (x - mean) * invstd
        gs = g * scale
        dx = invstd * (gs - gs.mean(axis=-1, keepdims=True) - xn * (gs * xn).mean(axis=-1, keepdims=True))
        node.state["np_dscale"] = (g * xn).reshape(-1, d).sum(axis=0)
        node.state["np_dbias"] = g.reshape(-1, d).sum(axis=0)
        return dx.astype(np.float32)

    def gpu_compute(self, node, iv, out, stream):
        g, x, scale = iv
        fwd = node.attrs["fwd"]
        st = node.state
        if "dscale" not in st:
            st["dscale"], st["dbias"] = _small(scale.shape, x.ctx), _small(scale.shape, x.ctx)
        G.layer_norm_grad(g, x, scale, fwd.state["mean"], fwd.state["invstd"], out, st["dscale"],
                          st["dbias"], stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(s[1])


_bnr, _bnrg = BatchNormReluOp(), BatchNormReluGradientOp()
_bn, _bng, _bngd, _bngs, _bngb = (BatchNormOp(), BatchNormGradientOp(), BatchNormGradDataOp(),
                                  BatchNormGradScaleOp(), BatchNormGradBiasOp())
_ln, _lng, _lng_data, _lng_scale, _lng_bias = (LayerNormOp(), LayerNormGradientOp(), BatchNormGradDataOp(),
                                               BatchNormGradScaleOp(), BatchNormGradBiasOp())


def batch_normalization_op(node_in, bn_scale, bn_bias, momentum=0.99, eps=0.01):
    return _bn(node_in, bn_scale, bn_bias, momentum, eps)


def batch_normalization_relu_op(node_in, bn_scale, bn_bias, momentum=0.99, eps=0.01):
    """Fused ``relu(batch_normalization(x))`` (extension: no counterpart op in the reference)."""
    return _bnr(node_in, bn_scale, bn_bias, momentum, eps)


def batch_normalization_gradient_op(out_gradient, in_node, bn_scale, eps, fwd=None):
    return _bng(out_gradient, in_node, bn_scale, eps, fwd)


def batch_normalization_gradient_of_data_op(bn_gradient, in_arr):
    return _bngd(bn_gradient, in_arr)


def batch_normalization_gradient_of_scale_op(bn_gradient, in_scale):
    return _bngs(bn_gradient, in_scale)


def batch_normalization_gradient_of_bias_op(bn_gradient, in_bias):
    return _bngb(bn_gradient, in_bias)


def layer_normalization_op(node_in, ln_scale, ln_bias, eps=1e-5):
    return _ln(node_in, ln_scale, ln_bias, eps)
